"""``Launcher`` and ``ResourceGroup`` of the ``dae`` API (reference python/dae/launcher.py): per-SM
instruction builders, countdown barriers with late-bound counts, the tensor-map table, resource groups
whose ids a device-side loop shifts per layer, and the launch through ``dae.runtime``.  Unlike the
reference it accepts every SM of the device (148 on a B200) instead of at most 132."""
import numpy as np
import torch

from . import runtime
from .instructions import *  # noqa: F401,F403
from .instructions import ComputeInstruction, Instruction, MemoryInstruction, TerminateC, TerminateM, TmaTensor
from .runtime import config, opcode
from .tma_utils import *  # noqa: F401,F403


def extract_compute_operator_names(launcher):
    names = []
    for b in launcher.builder:
        for inst in [*b.built_cinsts, *b.cinsts]:
            n = inst.compute_operator_name()
            if n not in names:
                names.append(n)
    return names


class SMInstructionBuilder:
    """The instruction lists of one SM.  `add` flattens lists, calls per-SM generators (anything callable
    gets the SM id) and sorts instructions into the compute and the memory stream."""

    def __init__(self, sm_id: int):
        self.sm_id = sm_id
        self.cinsts, self.minsts = [], []
        self.built_cinsts, self.built_minsts = [], []

    def add(self, inst):
        if inst is None:
            return
        if isinstance(inst, list):
            for sub in inst:
                self.add(sub)
        elif isinstance(inst, ComputeInstruction):
            self.cinsts.append(inst)
        elif isinstance(inst, MemoryInstruction):
            self.minsts.append(inst)
        elif callable(inst):
            self.add(inst(self.sm_id))
        else:
            raise ValueError("Unknown instruction type", inst)

    def add_compute(self, inst):
        self.cinsts.append(inst)

    def add_memory(self, inst):
        self.minsts.append(inst)

    def build(self, ctensor, cptrs, mtensor, mptrs):
        """Encodes the pending instructions into this SM's rings at the ring pointers, which advance."""
        assert len(self.cinsts) <= ctensor.shape[0] and len(self.minsts) <= mtensor.shape[0]
        cw = ctensor.numpy().view(np.uint16).reshape(ctensor.shape[0], 4)
        mw = mtensor.numpy().view(np.uint16).reshape(mtensor.shape[0], 8)
        for inst in self.cinsts:
            p = cptrs[self.sm_id]
            cw[p] = 0
            cw[p, 0] = inst.opcode_value()
            cw[p, 1:1 + len(inst.args)] = inst.args
            cptrs[self.sm_id] = (p + 1) % ctensor.shape[0]
        for inst in self.minsts:
            p = mptrs[self.sm_id]
            mw[p] = [inst.opcode, inst.size, inst.num_slots, inst.arg, *inst.cords]
            mptrs[self.sm_id] = (p + 1) % mtensor.shape[0]
        self.built_cinsts += self.cinsts
        self.built_minsts += self.minsts
        self.cinsts, self.minsts = [], []


class ResourceGroup:
    """Named tensor maps and barriers that exist once per repeat (layer).  Ids are laid out repeat-major, so
    a GROUP-flagged instruction reaches the next layer's resources by adding the group's width."""

    def __init__(self, name, repeat=1):
        self.name, self.repeat = name, repeat
        self.tmas, self.bars = {}, {}
        self.built, self.launcher = False, None
        self.tma_insts, self.bar_ids, self.bar_instances = {}, {}, {}

    def addTma(self, name: str, matList, tmaFn):
        if isinstance(matList, torch.Tensor):
            assert matList.dim() > 1, "matList must be a list of matrices or a 3D tensor"
            matList = [matList[i, ...] for i in range(matList.shape[0])]
        assert len(matList) == self.repeat, f"tmaList length {len(matList)} does not match group size {self.repeat}"
        assert name not in self.tmas, f"TMA with name {name} already exists in the group"
        self.tmas[name] = (matList, tmaFn)

    def addBarrier(self, name: str, bar_count=None):
        assert bar_count is None or isinstance(bar_count, int), "bar_count must be an int or None"
        assert name not in self.bars, f"Barrier with name {name} already exists in the group"
        self.bars[name] = {"count": bar_count, "late_bind": bar_count is None}

    def bindBarrier(self, name: str, bar_count: int):
        assert isinstance(bar_count, int), "bar_count must be an int"
        assert name in self.bars, f"Barrier with name {name} does not exist in the group"
        info = self.bars[name]
        if not info["late_bind"]:
            raise ValueError(f"Barrier {name} was declared with an eager count and cannot be rebound")
        if info["count"] is not None:
            raise ValueError(f"Barrier {name} has already been bound")
        info["count"] = bar_count
        if self.built:
            for bar_id in self.bar_instances[name]:
                self.launcher.set_bar(bar_id, bar_count)

    def bindBarriersFromCounts(self, bar_counts: dict):
        unresolved = []
        for name, info in self.bars.items():
            if not info["late_bind"] or info["count"] is not None:
                continue
            seen = {bar_counts[b] for b in self.bar_instances.get(name, []) if b in bar_counts}
            if not seen:
                unresolved.append(name)
            elif len(seen) > 1:
                raise ValueError(f"Barrier {name} observed inconsistent release counts: {sorted(seen)}")
            else:
                self.bindBarrier(name, seen.pop())
        if unresolved:
            raise ValueError(f"Could not infer release counts for late-bound barriers in group {self.name}: {unresolved}")

    def get_shift(self):
        return len(self.tmas), len(self.bars)

    def get(self, name: str):
        assert self.built, "ResourceGroup must be built before getting resource ids"
        if name in self.tmas:
            return self.tma_insts[name]
        if name in self.bars:
            return self.bar_ids[name]
        raise ValueError(f"Resource with name {name} not found in the group")

    def next(self, name: str, nnext: int = 1):
        return self.get(name) + len(self.bars) * nnext

    def over(self, name: str):
        return self.next(name, self.repeat)

    def __getitem__(self, name: str):
        return self.get(name)

    def range_bars(self):
        assert self.built, "ResourceGroup must be built before getting start id"
        lo, hi = min(self.bar_ids.values()), max(self.bar_ids.values())
        assert lo % 4 == 0, "bar ids must be aligned to 16 bytes for efficient encoding"
        return lo, (hi // 4 + 1) * 4

    def build(self, launcher):
        if self.built:
            return
        self.launcher = launcher
        for i in range(self.repeat):
            for name, (mats, fn) in self.tmas.items():
                inst = TmaTensor(launcher, mats[i])
                fn(inst)
                if self.repeat > 1:
                    inst.group()
                inst.annotation.update(group=self.name, tensor=name)
                if i == 0:
                    self.tma_insts[name] = inst
        # one more barrier instance than repeats: schedules address "the layer after the last" with next()/over()
        for i in range(self.repeat + 1):
            for name, info in self.bars.items():
                bar_id = launcher.new_bar(info["count"])
                self.bar_instances.setdefault(name, []).append(bar_id)
                if i == 0:
                    self.bar_ids[name] = bar_id
        while launcher.num_bars % 4:
            launcher.new_bar(0)
        self.built = True


class Launcher:
    def __init__(self, num_sms: int = 1, device="cuda"):
        self.smem_size = 202 * 1024     # what the reference asks for; the runtime sizes its own shared memory
        self.num_sms = num_sms
        self.device = device
        self.max_insts = config.max_insts
        self.builder = [SMInstructionBuilder(sm_id=i) for i in range(num_sms)]
        self.profile = torch.zeros((num_sms, config.num_profile_events), dtype=torch.uint64, device=device)
        self.cinsts = torch.zeros((num_sms, self.max_insts, 8), dtype=torch.uint8)
        self.minsts = torch.zeros((num_sms, self.max_insts, 16), dtype=torch.uint8)
        self.cptrs = [0] * num_sms
        self.mptrs = [0] * num_sms
        self.tmas = []
        self.need_instruction_build = True
        self.num_bars = 0
        self.bar_values = {}
        self._late_barriers_bound = False
        self.bars = torch.zeros(config.max_bars, 4, dtype=torch.uint8, device=device)
        self.bars_src = torch.zeros(config.max_bars, 4, dtype=torch.uint8, device=device)
        self.resource_groups = {"default": ResourceGroup("default")}
        self.timeout_ns = 0             # 0: the runtime's default budget for device-side waits (2 s)
        runtime.set_smem_size(self.smem_size)

    # ------------------------------------------------------------------ resources
    def add_group(self, name, size):
        assert name not in self.resource_groups, f"Resource group with name {name} already exists"
        self.resource_groups[name] = ResourceGroup(name, size)
        return self.resource_groups[name]

    def get_group(self, name="default"):
        assert name in self.resource_groups, f"Resource group with name {name} does not exist"
        return self.resource_groups[name]

    def build_groups(self):
        for group in self.resource_groups.values():
            group.build(self)

    def new_bar(self, value):
        bar_id = self.num_bars
        assert bar_id < config.max_bars, "out of global barriers"
        self.bar_values[bar_id] = value
        self.num_bars += 1
        return bar_id

    def set_bar(self, bar_id: int, value: int):
        assert bar_id in self.bar_values, f"bar_id {bar_id} does not exist"
        assert isinstance(value, int), "bar value must be an int"
        self.bar_values[bar_id] = value

    def new_tma(self, desc: torch.Tensor) -> int:
        assert len(self.tmas) < config.max_tmas, "out of tensor-map entries"
        self.tmas.append(desc)
        return len(self.tmas) - 1

    # ------------------------------------------------------------------ instructions
    def copy_cptrs(self):
        """Ring position the next compute instruction of every SM will get (the target of a LoopC)."""
        return [(self.cptrs[i] + len(self.builder[i].cinsts)) % self.max_insts for i in range(self.num_sms)]

    def copy_mptrs(self):
        return [(self.mptrs[i] + len(self.builder[i].minsts)) % self.max_insts for i in range(self.num_sms)]

    def build_instructions(self):
        if self.need_instruction_build:
            for i, b in enumerate(self.builder):
                b.build(self.cinsts[i], self.cptrs, self.minsts[i], self.mptrs)
            self.need_instruction_build = False

    def set_persistent(self, *tensors):
        stream = torch.cuda.current_stream().cuda_stream
        for t in tensors:
            runtime.set_cache_policy(t, stream, 1.0, 2, 0)

    def set_streaming(self, *tensors):
        stream = torch.cuda.current_stream().cuda_stream
        for t in tensors:
            if isinstance(t, torch.Tensor):
                runtime.set_cache_policy(t, stream, 0, 0, 1)
            elif isinstance(t, list):
                for x in t:
                    runtime.set_cache_policy(x, stream, 0, 0, 1)
            else:
                raise ValueError("tensor must be a torch.Tensor or a list of torch.Tensor")

    def i(self, *insts):
        """Adds instructions (or lists, or per-SM generators) to every SM's builder."""
        for inst in insts:
            for b in self.builder:
                b.add(inst)
        self.need_instruction_build = True

    def s(self, *schedules):
        self.i(*schedules, TerminateC(), TerminateM())

    def collect_barrier_release_counts(self, *insts):
        counts = {}

        def visit(x):
            if isinstance(x, list):
                for y in x:
                    visit(y)
            elif x is not None and hasattr(x, "collect_barrier_release_counts"):
                for bar_id, n in x.collect_barrier_release_counts().items():
                    counts[bar_id] = counts.get(bar_id, 0) + n
        visit(list(insts))
        return counts

    def bind_late_barrier_counts(self, *insts):
        if self._late_barriers_bound:
            return
        counts = self.collect_barrier_release_counts(*insts)
        for group in self.resource_groups.values():
            group.bindBarriersFromCounts(counts)
        self._late_barriers_bound = True

    def num_insts(self):
        ci = sum(len(b.cinsts) for b in self.builder)
        mi = sum(len(b.minsts) for b in self.builder)
        return ci / self.num_sms, mi / self.num_sms

    def compute_operator_names(self):
        return extract_compute_operator_names(self)

    # ------------------------------------------------------------------ launch
    def launch(self):
        self.build_instructions()
        supported = getattr(runtime, "supported_compute_ops", None)
        if supported is not None:
            needed = self.compute_operator_names()
            missing = [n for n in needed if n not in set(supported)]
            if missing:
                raise ValueError("Launcher requires compute operators that are not compiled into dae.runtime: "
                                 f"{missing}. Rebuild with DAE_COMPUTE_OPS={','.join(needed)} or a superset.")
        unbound = [b for b, v in self.bar_values.items() if v is None]
        if unbound:
            raise ValueError(f"Cannot launch with unbound barrier counts: {unbound}")
        runtime.validate_streams(self.num_sms, self.max_insts, self.cinsts.numpy(), self.minsts.numpy())
        cinsts = self.cinsts.to(self.device).view(self.num_sms * self.max_insts, 8)
        minsts = self.minsts.to(self.device).view(self.num_sms * self.max_insts, 16)
        stream = torch.cuda.current_stream().cuda_stream
        image = torch.zeros(config.max_bars, dtype=torch.int32)
        for bar_id, value in self.bar_values.items():
            image[bar_id] = value
        self.bars.view(torch.int32).view(-1).copy_(image)
        self.bars_src.view(torch.int32).view(-1).copy_(image)
        tma = torch.stack(self.tmas).to(self.device) if self.tmas else torch.zeros((4, 128), dtype=torch.uint8,
                                                                                   device=self.device)
        profile = self.profile.view(torch.uint8).view(self.num_sms * config.num_profile_events, 8)
        runtime.set_cache_policy(self.bars, stream, 1, 2, 0)
        runtime.set_cache_policy(tma, stream, 1, 2, 0)
        ret = runtime.launch_dae(self.num_sms, self.smem_size, cinsts, minsts, tma, self.bars.view(torch.int32).view(-1),
                                 profile.view(torch.int64).view(-1), stream, timeout_ns=self.timeout_ns,
                                 insts_per_sm=self.max_insts)
        assert ret == 0

    def bench(self, iterations: int = 100, total_bytes=None, total_flops=None):
        """Launches `iterations` times and reads the device-side start / end stamps of every SM."""
        per_sm = np.zeros(self.num_sms, dtype=np.float64)
        span = 0.0
        for _ in range(iterations):
            self.launch()
            t = self.profile[:, 0:2].cpu().view(torch.int64).numpy()
            per_sm += t[:, 1] - t[:, 0]
            span += float(t[:, 1].max() - t[:, 0].min())
        avg_ns = float(per_sm.mean() / iterations)
        print(f"Benchmark Results on {self.num_sms} SMs and {iterations} iterations:")
        print(f"Average duration (ns): {avg_ns:.2f}")
        print(f"Average execution time (ns): {span / iterations:.2f}")
        if total_bytes is not None:
            print(f"Effective Bandwidth (GB/s): {total_bytes / (avg_ns / 1e9) / (1024 ** 3):.2f}")
        if total_flops is not None:
            print(f"Effective GFLOPS: {total_flops / avg_ns / 1e6:.2f}")
        return avg_ns
