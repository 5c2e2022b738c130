"""Schedule combinators of the ``dae`` API (reference python/dae/schedule.py): a schedule is a per-SM
instruction generator.  ``place(n, base)`` binds it to SMs base..base+n-1, ``bar(role, id)`` names the
barrier a role waits for or releases, ``collect_barrier_release_counts()`` tells the launcher how often
each barrier is counted down so that late-bound barriers get their initial values."""
import copy as pycopy
import warnings

import torch

from .launcher import *  # noqa: F401,F403
from .instructions import (RawAddress, RegLoad, RepeatM, SILU_MUL_SHARED_BF16_K_4096_INTER,
                           SILU_MUL_SHARED_BF16_K_64_SW128, TmaLoad1D, TmaStore1D, Copy,
                           select_attention_decode_instruction, select_rms_smem_instruction)
from .runtime import *  # noqa: F401,F403


class Schedule:
    def __init__(self):
        self.num_sms = None
        self.base_sm = 0
        self._bars = {}

    def _clone(self):
        clone = pycopy.copy(self)
        clone._bars = dict(self._bars)
        return clone

    def _on_place(self):
        pass

    def place(self, num_sms: int, base_sm: int = 0):
        clone = self._clone()
        clone.num_sms, clone.base_sm = num_sms, base_sm
        clone._on_place()
        return clone

    def bar(self, role: str, bar_id: int):
        self._bars[role] = bar_id
        return self

    def _bar(self, role: str):
        return self._bars.get(role)

    def _require_placed(self):
        if self.num_sms is None:
            raise ValueError(f"{self.__class__.__name__} must be placed before querying barrier release counts")

    def _bar_release_if_present(self, role: str, count: int):
        if self._bar(role) is None:
            return 0
        self._require_placed()
        return count

    def bar_release_count(self, role: str):
        return 0

    def collect_barrier_release_counts(self):
        counts = {}
        for role, bar_id in self._bars.items():
            n = self.bar_release_count(role)
            if n > 0:
                counts[bar_id] = counts.get(bar_id, 0) + n
        return counts

    def map_sm(self, sm: int):
        """Device SM id -> index inside this schedule's placement, -1 outside it."""
        if self.num_sms is None:
            raise ValueError(f"{self.__class__.__name__} must be placed before scheduling")
        local = sm - self.base_sm
        return local if 0 <= local < self.num_sms else -1

    def schedule(self, sm: int):
        raise NotImplementedError("Schedule.schedule() must be implemented by subclass")

    def __call__(self, sm: int):
        return self.schedule(self.map_sm(sm))


class ListSchedule(Schedule):
    """Several schedules run one after the other on the same SMs.  A barrier role named on the list goes to the
    first member (lead_bars), the last member (tail_bars) or both."""

    def __init__(self, items, lead_bars=None, tail_bars=None, warn_boundary_bars=False):
        super().__init__()
        self.items = list(items)
        self.lead_bars = set(lead_bars or ())
        self.tail_bars = set(tail_bars or ())
        self.warn_boundary_bars = warn_boundary_bars
        self._warned_boundary_roles = set()

    def _clone(self):
        clone = super()._clone()
        clone.items = [it._clone() if isinstance(it, Schedule) else it for it in self.items]
        clone.lead_bars, clone.tail_bars = set(self.lead_bars), set(self.tail_bars)
        clone._warned_boundary_roles = set(self._warned_boundary_roles)
        return clone

    def _schedule_items(self):
        return [it for it in self.items if isinstance(it, Schedule)]

    def warn_on_boundary_bars(self, enable=True):
        self.warn_boundary_bars = enable
        return self

    def _apply_boundary_bars(self):
        members = self._schedule_items()
        if not members:
            return
        first, last = members[0], members[-1]
        for role, bar_id in self._bars.items():
            boundary = role in self.lead_bars or role in self.tail_bars
            if self.warn_boundary_bars and len(members) > 1 and boundary and role not in self._warned_boundary_roles:
                warnings.warn(f"ListSchedule bar('{role}', ...) only applies to boundary schedule(s); "
                              "this may be insufficient for interior dependencies", stacklevel=3)
                self._warned_boundary_roles.add(role)
            if role in self.lead_bars:
                first.bar(role, bar_id)
            if role in self.tail_bars:
                last.bar(role, bar_id)
            if not boundary:
                if first is not last:
                    raise ValueError(f"ListSchedule cannot route bar role '{role}'")
                first.bar(role, bar_id)

    def place(self, num_sms: int, base_sm: int = 0):
        clone = self._clone()
        clone.num_sms, clone.base_sm = num_sms, base_sm
        clone.items = [it.place(num_sms, base_sm) if isinstance(it, Schedule) else it for it in clone.items]
        clone._apply_boundary_bars()
        return clone

    def bar(self, role: str, bar_id: int):
        super().bar(role, bar_id)
        self._apply_boundary_bars()
        return self

    def __call__(self, sm: int):
        return [it(sm) if callable(it) else it for it in self.items]

    def __getitem__(self, idx):
        return self.items[idx]

    def __iter__(self):
        return iter(self.items)

    def __len__(self):
        return len(self.items)

    def bar_release_count(self, role: str):
        return sum(it.bar_release_count(role) for it in self._schedule_items())

    def collect_barrier_release_counts(self):
        counts = {}
        for it in self._schedule_items():
            for bar_id, n in it.collect_barrier_release_counts().items():
                counts[bar_id] = counts.get(bar_id, 0) + n
        return counts


def interleave(*schedules):
    return [s for group in zip(*schedules) for s in group]


def _released_by_every_sm(role_name):
    """bar_release_count for schedules whose `role_name` barrier is counted down once per placed SM."""
    def bar_release_count(self, role: str):
        return self._bar_release_if_present(role, self.num_sms) if role == role_name else 0
    return bar_release_count


class SchedCopy(Schedule):
    """One load -> COPY -> store per SM; tmas = (load template, store template), addressed by SM index."""

    def __init__(self, tmas, size=None, before_copy=None, count=1):
        super().__init__()
        self.tmas, self.count, self.before_copy = tmas, count, before_copy
        if size is None:
            assert tmas[0].size == tmas[1].size, "Size must be specified when load and store TMA sizes do not match"
            size = tmas[0].size
        self.size = size

    def schedule(self, sm: int):
        if sm < 0:
            return []
        load, store = (t.cord(sm) for t in self.tmas)
        if self.before_copy is not None:
            load.jump()         # the instruction in front (an embedding indirection) is a one-trip loop header
        return [Copy(1, size=self.size), self.before_copy, load.bar(self._bar("load")), store.bar(self._bar("store"))]

    bar_release_count = _released_by_every_sm("store")


class SchedRope(Schedule):
    def __init__(self, Atom, tmas):
        super().__init__()
        self.Atom, self.tmas = Atom, tmas

    def schedule(self, sm: int):
        if sm < 0:
            return []
        table, load, store = (t.cord(sm) for t in self.tmas)
        return [self.Atom(), table, load, store.bar(self._bar("store")).group()]

    bar_release_count = _released_by_every_sm("store")


class SchedGemv(Schedule):
    """y[N, M] = x[N, K] W[M, K]^T in tiles of Atom.MNK: SM s owns rows (s mod M/TileM) * TileM and the K-slice
    number s div (M/TileM) of `fold` slices (fold > 1: the store must be a reduce-add).  Per tile group the
    activation tile is loaded once and n_batch weight tiles follow it."""

    def __init__(self, Atom, MNK, tmas, fold=None, exec=True, prefetch=True, group=True):
        super().__init__()
        assert len(MNK) == 3, "MNK must be a tuple of 3 dimensions"
        self.Atom, self.tmas = Atom, tmas
        base, size = [], []
        for dim in MNK:
            if isinstance(dim, int):
                base.append(0)
                size.append(dim)
            elif isinstance(dim, tuple) and len(dim) == 2:
                base.append(dim[0])
                size.append(dim[1])
            else:
                raise ValueError(f"Invalid MNK dimension: {dim}")
        self.MNK, self.MNK_base = size, base
        self.fold, self.exec, self.prefetch, self.group = fold, exec, prefetch, group
        self.sm_per_fold = self.k_per_fold = None

    def _on_place(self):
        TileM = self.Atom.MNK[0]
        M, _, K = self.MNK
        if self.fold is None:
            assert self.num_sms % (M // TileM) == 0, (
                f"SMS must be multiple of M tiles when auto folding, got SMS={self.num_sms}, M={M}, TileM={TileM}")
            self.fold = self.num_sms // (M // TileM)
        self.sm_per_fold = self.num_sms // self.fold
        self.k_per_fold = K // self.fold
        self.validate()

    def validate(self):
        TileM, TileN, TileK = self.Atom.MNK
        M, N, K = self.MNK
        group_k = TileK * self.Atom.n_batch
        assert K % TileK == 0 and M % TileM == 0 and N % TileN == 0
        assert self.MNK_base[1] == 0, "N dimension must start from 0 for current schedule design"
        assert self.num_sms % self.fold == 0 and K % self.fold == 0
        assert self.sm_per_fold == M // TileM, "Invalid fold for given SMS and M size"
        assert self.k_per_fold % TileK == 0, "Invalid fold for given K size"
        assert self.k_per_fold % group_k == 0 and self.k_per_fold >= group_k, (
            f"Invalid fold for {self.Atom.__name__}: k_per_fold={self.k_per_fold} must be a positive multiple of "
            f"TileK * n_batch = {TileK} * {self.Atom.n_batch} = {group_k}")
        assert len(self.tmas) == 3, "Expect at 3 TMA tensors: loadA, loadB, storeC"
        if self.fold > 1:
            assert self.tmas[-1].mode == "reduce", f"storeC must be reduction mode when fold > 1, got mode {self.tmas[-1].mode}"

    def schedule(self, sm: int):
        if sm < 0:
            return []
        TileM, _, TileK = self.Atom.MNK
        n_batch = self.Atom.n_batch
        loadA, loadB, storeC = self.tmas
        m = self.MNK_base[0] + (sm % self.sm_per_fold) * TileM
        k = self.MNK_base[2] + (sm // self.sm_per_fold) * self.k_per_fold
        step = TileK * n_batch
        grouped_load = self.group and self._bar("load") is not None
        grouped_store = self.group and self._bar("store") is not None
        body = [(loadB.cord(0, k).group(grouped_load), loadB.cord2tma(0, step))]
        body += [(loadA.cord(m, k + TileK * i).group(grouped_load), loadA.cord2tma(0, step)) for i in range(n_batch)]
        return [
            self.Atom(self.k_per_fold // TileK),
            RepeatM.onSync(0, self._bar("load"), self.k_per_fold // step, *body, asyncPort=self.prefetch),
            storeC.cord(0, m).bar(self._bar("store")).group(grouped_store),
        ]

    def split(self, dim: int, div: int):
        """`div` schedules that each cover one part of dimension `dim` (0: M, 2: K), run back to back."""
        assert dim in (0, 1, 2), "dim must be 0 (M), 1 (N), or 2 (K)"
        assert self.MNK[dim] % div == 0, "Cannot split dimension that is not divisible by div"
        part = self.MNK[dim] // div
        pieces = []
        for i in range(div):
            dims = [(b, s) for b, s in zip(self.MNK_base, self.MNK)]
            dims[dim] = (self.MNK_base[dim] + i * part, part)
            pieces.append(SchedGemv(self.Atom, tuple(dims), self.tmas, fold=self.fold, prefetch=self.prefetch,
                                    group=self.group))
        out = ListSchedule(pieces, lead_bars={"load"}, tail_bars={"store"})
        out._bars = dict(self._bars)
        if self.num_sms is not None:
            return out.place(self.num_sms, self.base_sm)
        out._apply_boundary_bars()
        return out

    def split_M(self, div: int):
        return self.split(0, div)

    def split_K(self, div: int):
        return self.split(2, div)

    def no_prefetch(self):
        self.prefetch = False
        return self

    bar_release_count = _released_by_every_sm("store")


class SchedRMSShared(Schedule):
    """RMSNorm of num_token rows in shared memory; tmas = (weight, input template, output template)."""

    def __init__(self, num_token, epsilon, tmas, hidden_size=None, group=True, embedding=None):
        super().__init__()
        self.num_token, self.epsilon, self.tmas = num_token, epsilon, tmas
        self.hidden_size, self.group, self.embedding = hidden_size, group, embedding

    def _on_place(self):
        assert self.num_token % self.num_sms == 0, "Number of tokens must be divisible by number of SMs"
        self.workload_per_sm = self.num_token // self.num_sms

    def _resolve_hidden_size(self):
        if self.hidden_size is not None:
            return self.hidden_size
        weight = self.tmas[0]
        if hasattr(weight, "size") and weight.size % 2 == 0:
            return weight.size // 2
        raise ValueError("SchedRMSShared requires hidden_size or a byte-sized weight TMA")

    def schedule(self, sm):
        if sm < 0:
            return []
        hidden = self._resolve_hidden_size()
        offset = hidden * 2 * sm * self.workload_per_sm
        weight, load, store = self.tmas
        load = load.cord(offset).bar(self._bar("input")).group(self.group)
        store = store.cord(offset).bar(self._bar("output")).group(self.group)
        if self.embedding is not None:
            load.jump()
        return [select_rms_smem_instruction(hidden)(self.workload_per_sm, self.epsilon), weight.group(), self.embedding,
                load, store]

    bar_release_count = _released_by_every_sm("output")


class SchedSmemSiLUInterleaved(Schedule):
    """silu(gate) * up for whole rows held in shared memory, one task per token."""

    def __init__(self, num_token, gate_glob, up_glob, out_glob):
        super().__init__()
        self.num_token, self.gate_glob, self.up_glob, self.out_glob = num_token, gate_glob, up_glob, out_glob

    def _on_place(self):
        assert self.num_token % self.num_sms == 0, "Number of tokens must be divisible by number of SMs"
        self.tokens_per_sm = self.num_token // self.num_sms

    def schedule(self, sm):
        if sm < 0:
            return []
        insts = []
        first = sm * self.tokens_per_sm
        for i in range(first, first + self.tokens_per_sm):
            gate = TmaLoad1D(self.gate_glob[i])
            if i == first:
                gate = gate.bar(self._bar("input")).group()
            insts += [SILU_MUL_SHARED_BF16_K_4096_INTER(1),
                      TmaStore1D(self.out_glob[i]).bar(self._bar("output")).group(), gate, TmaLoad1D(self.up_glob[i])]
        return insts

    def bar_release_count(self, role: str):
        return self._bar_release_if_present(role, self.num_token) if role == "output" else 0


class SchedRegSiLUFused(Schedule):
    """silu(gate) * up on the two result tiles a gate and an up projection left in registers (RegStore)."""

    def __init__(self, num_token, store_tma, reg_gate, reg_up, base_offset, stride):
        super().__init__()
        self.num_token, self.store_tma = num_token, store_tma
        self.reg_gate, self.reg_up, self.base_offset, self.stride = reg_gate, reg_up, base_offset, stride

    def schedule(self, sm):
        if sm < 0:
            return []
        return [SILU_MUL_SHARED_BF16_K_64_SW128(self.num_token),
                self.store_tma.cord(0, self.base_offset + sm * self.stride).bar(self._bar("output")).group(),
                RegLoad(self.reg_gate), RegLoad(self.reg_up)]

    bar_release_count = _released_by_every_sm("output")


class SchedArgmax(Schedule):
    """Greedy token ids: every SM reduces its chunk of the logits to (value, index); SM t < num_token then reduces
    token t's partial results over all SMs."""

    def __init__(self, num_token, logits_slice, num_slice, AtomPartial, AtomReduce, matLogits, matOutVal, matOutIdx,
                 matFinalOut):
        super().__init__()
        self.num_token, self.logits_slice, self.num_slice = num_token, logits_slice, num_slice
        self.AtomPartial, self.AtomReduce = AtomPartial, AtomReduce
        self.matLogits, self.matOutVal, self.matOutIdx, self.matFinalOut = matLogits, matOutVal, matOutIdx, matFinalOut

    def _on_place(self):
        self.validate()

    def validate(self):
        assert len(self.matLogits) == self.num_slice, "Number of logits slices must match vocab size and slice size"
        assert self.matOutVal.shape == (self.num_token, self.num_sms)
        assert self.matOutIdx.shape == (self.num_token, self.num_sms)
        assert self.matFinalOut.shape == (self.num_token,)
        assert self.num_sms % self.num_slice == 0, "Number of SMs must be divisible by number of slices"
        chunk = self.logits_slice // (self.num_sms // self.num_slice)
        assert self.logits_slice % chunk == 0
        for atom in (self.AtomPartial, self.AtomReduce):
            assert atom.CHUNK_SIZE == chunk, f"{atom.__name__} chunk size mismatch, expected {chunk}, got {atom.CHUNK_SIZE}"
            assert atom.SMS == self.num_sms, f"{atom.__name__} SMS mismatch, expected {self.num_sms}, got {atom.SMS}"
        assert self.AtomPartial.I_STRIDE == self.logits_slice

    def schedule(self, sm):
        if sm < 0:
            return []
        per_slice = self.num_sms // self.num_slice
        chunk = self.logits_slice // per_slice
        insts = [
            self.AtomPartial(self.num_token),
            RawAddress(self.matLogits[sm // per_slice][0, (sm % per_slice) * chunk], 24).bar(self._bar("load")),
            RawAddress(self.matOutVal[0, sm], 25).bar(self._bar("val")).writeback(),
            RawAddress(self.matOutIdx[0, sm], 26).bar(self._bar("idx")).writeback(),
        ]
        if sm < self.num_token:
            insts += [
                self.AtomReduce(1),
                RawAddress(self.matOutVal[sm], 27).bar(self._bar("val")),
                RawAddress(self.matOutIdx[sm], 28).bar(self._bar("idx")),
                RawAddress(self.matFinalOut[sm], 29).bar(self._bar("final")).writeback(),
            ]
        return insts

    def bar_release_count(self, role: str):
        if role in ("val", "idx"):
            return self._bar_release_if_present(role, self.num_sms)
        if role == "final":
            return self._bar_release_if_present(role, min(self.num_token, self.num_sms))
        return 0


class SchedAttentionDecoding(Schedule):
    """Decode attention (one query token per request), one SM per (request, head): the SM's stream is the
    attention instruction, [the side input row (q-norm | k-norm | rope) of the token's position and the
    k-store row, for the fused QK-norm + RoPE path], the Q tile behind the "q" barrier, a REPEAT over the
    first seq_len / block - 1 (K block, V block) pairs, the last pair with its K behind the "k" barrier (only
    the last block holds a row produced in this step), and the output row store releasing "o".
    Mirrors python/dae/schedule.py:250-325 of the reference."""

    def __init__(self, reqs: int, seq_len: int, KV_BLOCK_SIZE: int, NUM_KV_HEADS: int, matO: torch.Tensor, tmas,
                 side_input=None, k_store=None, token_pos=None):
        super().__init__()
        self.reqs, self.seq_len, self.block_size, self.num_heads = reqs, seq_len, KV_BLOCK_SIZE, NUM_KV_HEADS
        self.matO, self.tmas = matO, tmas
        self.side_input, self.k_store, self.token_pos = side_input, k_store, token_pos
        self.required_sms = reqs * NUM_KV_HEADS
        self.AttentionInst = select_attention_decode_instruction(matO.shape[-1])
        self.use_qwen_fused_qk = side_input is not None
        if self.use_qwen_fused_qk and (k_store is None or token_pos is None):
            raise ValueError("SchedAttentionDecoding requires side_input, k_store, and token_pos together for the "
                             "fused Qwen path")

    def _on_place(self):
        assert self.num_sms == self.required_sms, (
            f"SchedAttentionDecoding requires {self.required_sms} SMs, got {self.num_sms}")

    def schedule(self, sm: int):
        if sm < 0:
            return []
        req, head = divmod(sm, self.num_heads)
        head_dim = self.matO.shape[-1]
        tQ, tK, tV = self.tmas
        n_blocks = (self.seq_len + self.block_size - 1) // self.block_size
        last_len = self.seq_len % self.block_size or self.block_size
        fused = self.use_qwen_fused_qk
        insts = [self.AttentionInst(n_blocks, last_len, need_norm=fused, need_rope=fused)]
        if fused:
            insts += [self.side_input.cord(self.token_pos * 3 * head_dim).group(),
                      self.k_store[req].cord((self.token_pos * self.num_heads + head) * head_dim).group()]
        last0 = self.block_size * (n_blocks - 1)
        insts += [
            tQ.cord(req, head).bar(self._bar("q")).group(),
            RepeatM.on(n_blocks - 1,
                       [tK.cord(req, 0, head, 0).group(), tK.cord2tma(0, self.block_size, 0, 0)],
                       [tV.cord(req, 0, head, 0).group(), tV.cord2tma(0, self.block_size, 0, 0)]),
            tK.cord(req, last0, head, 0).bar(self._bar("k")).group(),
            tV.cord(req, last0, head, 0).group(),
            TmaStore1D(self.matO[req, head, ...], numSlots=2).bar(self._bar("o")).group(),
        ]
        return insts

    def bar_release_count(self, role: str):
        if role != "o":
            return 0
        return self._bar_release_if_present(role, self.num_sms)
