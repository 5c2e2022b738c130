"""Name-mangled compute-op families (reference python/dae/op_families.py): a family member is named
``OP_<FAMILY>__<FIELD>_<value>__...`` and must exist in the runtime's opcode table to be launched."""
from dataclasses import dataclass
from functools import lru_cache

from . import runtime
from .op_family_specs import ComputeFamilyDefinition, parse_comp_family_runtime_specs


@dataclass(frozen=True)
class ComputeOpFamilyRef:
    canonical_name: str


@lru_cache(maxsize=1)
def family_definitions():
    specs = getattr(runtime, "compute_family_specs", None)
    if specs is None:
        raise ValueError("dae.runtime does not export compute_family_specs")
    defs = parse_comp_family_runtime_specs(list(specs))
    if not defs:
        raise ValueError("dae.runtime exported no compute family specs")
    return defs


def family_definition(family: str) -> ComputeFamilyDefinition:
    try:
        return family_definitions()[family.upper()]
    except KeyError as exc:
        raise ValueError(f"Unknown compute family definition for {family}") from exc


def _check(d: ComputeFamilyDefinition, values: dict):
    for f in d.fields:
        v, c = values[f], d.constraints
        if f + "_FIXED" in c and v != c[f + "_FIXED"]:
            raise ValueError(f"Unsupported {d.family} {f.lower()}={v}; expected {c[f + '_FIXED']}")
        if f + "_MULTIPLE" in c and (v <= 0 or v % c[f + "_MULTIPLE"]):
            raise ValueError(f"Unsupported {d.family} {f.lower()}={v}; expected a positive multiple of {c[f + '_MULTIPLE']}")
        if f + "_MIN" in c and v < c[f + "_MIN"]:
            raise ValueError(f"Unsupported {d.family} {f.lower()}={v}; expected >= {c[f + '_MIN']}")
        if f + "_MAX" in c and v > c[f + "_MAX"]:
            raise ValueError(f"Unsupported {d.family} {f.lower()}={v}; expected <= {c[f + '_MAX']}")


def _mangle(d: ComputeFamilyDefinition, values: dict) -> str:
    return "__".join([f"OP_{d.family}"] + [f"{f}_{values[f]}" for f in d.fields])


def family_ref(family: str, /, **values) -> ComputeOpFamilyRef:
    d = family_definition(family)
    vals = {k.upper(): int(v) for k, v in values.items()}
    missing = [f for f in d.fields if f not in vals]
    extra = [f for f in vals if f not in d.fields]
    if missing:
        raise ValueError(f"Missing {family} family fields: {missing}")
    if extra:
        raise ValueError(f"Unexpected {family} family fields: {extra}")
    _check(d, vals)
    return ComputeOpFamilyRef(_mangle(d, vals))


def family_spec_by_name(name):
    if not isinstance(name, str) or not name.startswith("OP_"):
        return None
    head, *tokens = name.split("__")
    if not tokens:
        return None
    try:
        d = family_definition(head[3:])
    except ValueError:
        return None
    if len(tokens) != len(d.fields):
        raise ValueError(f"Malformed {d.family} compute-op name: {name}. Expected fields {d.fields}.")
    vals = {}
    for f, tok in zip(d.fields, tokens):
        if not tok.startswith(f + "_"):
            raise ValueError(f"Malformed {d.family} compute-op name: {name}. Expected token starting with {f}_.")
        try:
            vals[f] = int(tok[len(f) + 1:])
        except ValueError as exc:
            raise ValueError(f"Malformed {d.family} compute-op name: {name}. {f} must be an integer.") from exc
    _check(d, vals)
    return {"name": _mangle(d, vals), "family": d.family.lower(), **{f.lower(): v for f, v in vals.items()}}


def is_registered_family_name(name) -> bool:
    return family_spec_by_name(name) is not None


def validate_family_name(name):
    if not isinstance(name, str):
        raise TypeError(f"Expected family opcode name as str, got {type(name).__name__}")
    if not is_registered_family_name(name):
        raise ValueError(f"Unknown dynamic compute-op family name: {name}")
    return name


def family_name(ref) -> str:
    return ref.canonical_name if isinstance(ref, ComputeOpFamilyRef) else validate_family_name(ref)


__all__ = ["ComputeFamilyDefinition", "ComputeOpFamilyRef", "family_definition", "family_definitions", "family_name",
           "family_ref", "family_spec_by_name", "is_registered_family_name", "validate_family_name"]
