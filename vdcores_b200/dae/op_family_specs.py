"""Parsing of compute-op family definitions (reference python/dae/op_family_specs.py): a family is a
list of integer fields plus constraints ``<FIELD>_FIXED / _MULTIPLE / _MIN / _MAX``, written as
``FIELDS=M|N|K, M_MULTIPLE=64, ...``."""
from dataclasses import dataclass
import re


@dataclass(frozen=True)
class ComputeFamilyDefinition:
    family: str
    fields: tuple
    constraints: dict


def parse_comp_family_definition(family: str, raw_definition: str) -> ComputeFamilyDefinition:
    items = {}
    for token in (t.strip() for t in raw_definition.split(",")):
        if "=" not in token:
            raise ValueError(f"Malformed family definition token for {family}: {token}")
        key, value = token.split("=", 1)
        items[key.strip().upper()] = value.strip()
    if "FIELDS" not in items:
        raise ValueError(f"Malformed family definition for {family}: missing FIELDS")
    fields = tuple(f.strip().upper() for f in items.pop("FIELDS").split("|"))
    return ComputeFamilyDefinition(family.upper(), fields, {k: int(v) for k, v in items.items()})


_LINE = re.compile(r"^\s*DAE_DEFINE_COMP_FAMILY\(\s*(\w+)\s*,\s*(.+)\)\s*(?://.*)?$")


def parse_comp_family_registry_lines(lines):
    out = {}
    for line in lines:
        m = _LINE.match(line.strip())
        if m:
            d = parse_comp_family_definition(*m.groups())
            out[d.family] = d
    return out


def parse_comp_family_runtime_specs(specs):
    out = {}
    for spec in specs:
        d = parse_comp_family_definition(str(spec["family"]), str(spec["definition"]))
        out[d.family] = d
    return out


__all__ = ["ComputeFamilyDefinition", "parse_comp_family_definition", "parse_comp_family_registry_lines",
           "parse_comp_family_runtime_specs"]
