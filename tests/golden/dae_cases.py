"""Instruction-stream cases built through the ``dae`` Python API, written once and run against two
implementations of that API: the reference's python/dae (by make_dae_golden.py, here in this container)
and this repository's vdcores_b200/dae (by tests/test_dae_api_cpu.py, anywhere).  Each case returns the
encoded bytes of the instructions it produced; the two must agree byte for byte.

No GPU is needed: tensors are stand-ins that only know their shape, strides and a made-up device
address, and tensor-map descriptors are replaced by a record of the arguments they were built from."""
import numpy as np
import torch


class FakeDevice:
    type = "cuda"


class FakeTensor:
    """Shape, strides, element size and address of a contiguous device tensor (or a view into one)."""
    device = FakeDevice()

    def __init__(self, shape, es=2, addr=0x7f00_0000_0000, strides=None):
        self.shape = tuple(shape)
        self._es = es
        self._addr = addr
        if strides is None:
            strides, acc = [], 1
            for s in reversed(self.shape):
                strides.insert(0, acc)
                acc *= s
        self._strides = tuple(strides)

    def dim(self):
        return len(self.shape)

    def stride(self, i=None):
        return self._strides if i is None else self._strides[i]

    def view(self, *shape):
        return FakeTensor(shape, self._es, self._addr)

    def numel(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    def element_size(self):
        return self._es

    def data_ptr(self):
        return self._addr

    def is_contiguous(self):
        return True

    def __getitem__(self, idx):
        if not isinstance(idx, tuple):
            idx = (idx,)
        idx = [i for i in idx if i is not Ellipsis]
        off = sum(i * s for i, s in zip(idx, self._strides))
        return FakeTensor(self.shape[len(idx):], self._es, self._addr + off * self._es, self._strides[len(idx):])


def fake_build_tma_desc(base, shape, strides_bytes, box_dim, elem_strides, swizzle_bytes=0, interleave=0):
    """Stands in for runtime.build_tma_desc: a 128-byte record of the arguments (the recipe under test)."""
    words = [base.data_ptr(), base.element_size(), len(shape), *shape, *strides_bytes, *box_dim, *elem_strides,
             swizzle_bytes, interleave]
    rec = np.zeros(16, dtype=np.int64)
    rec[:len(words)] = words[:16]
    return torch.from_numpy(rec.view(np.uint8).copy())


def encode(insts):
    """Flattens nested lists / None and concatenates the encodings (8 bytes compute, 16 bytes memory)."""
    out = []

    def walk(x):
        if x is None:
            return
        if isinstance(x, list):
            for y in x:
                walk(y)
            return
        out.append(x.tensor().numpy().copy().reshape(-1))
    walk(insts)
    return np.concatenate(out) if out else np.zeros(0, dtype=np.uint8)


def build_cases(D):
    """D: a namespace with the names of dae.launcher / dae.schedule / dae.model star-imports."""
    cases = {}
    T = FakeTensor
    op = D.opcode
    # ---------------------------------------------------------------- single instructions and flags
    mi = D.MemoryInstruction
    cases["mem_flags"] = encode([
        mi(op.OP_ALLOC_TMA_LOAD_1D, 2, 0, 16384, address=0x1234_5678_9ABC).port(1).bar(37).group().jump(),
        mi(op.OP_ALLOC_WB_TMA_STORE_2D, 1, 17, 1024, cords=[64, 8]).bar(5).writeback(),
        mi(op.OP_ALLOC_TMA_LOAD_3D, 4, 3, 32768, cords=[0, 128, 7]).delta([0, 0, 4]).copy(),
        mi(op.OP_ALLOC_TMA_LOAD_1D, 1, 0, 8192, address=0xFFF0).delta(0x20),
        D.TerminateM(), D.IssueBarrier(41), D.LoopM(32, 11, bar_shift=12, tma_shift=9, reg=3),
        D.RepeatM(7, reg=2, reg_end=6, delta_addr=0x8000), D.RepeatM(3, delta_cords=[0, 4, 0, 1]),
        D.RawAddress(T((8,), 4), 27), D.RawAddress(T((8,), 4), 24).bar(9).writeback(),
        D.CC0(T((16,), 8), 3, hidden_size=4096), D.CC0(T((16,), 8), 0, hidden_size=5120),
        D.RegStore(1, size=1024), D.RegStore(2, T((64, 8))), D.RegLoad(1), D.RegLoad(0, slot_id=3),
        D.TmaLoad1D(T((4096,))), D.TmaLoad1D(T((4, 4096)), bytes=2048, numSlots=2).cord(4096),
        D.TmaStore1D(T((2, 64, 128))[1]).cord(256).bar(3).group(),
    ])
    cases["compute"] = encode([
        D.TerminateC(), D.Dummy(5), D.Copy(3, 8192), D.LoopC(32, 17), D.Gemv_M64N8(16), D.Gemv_M64N8(8, 0, True),
        D.Gemv_M64N8B2(4), D.Gemv_M64N8_MMA(16), D.RMS_NORM_F16_K_4096_SMEM(8, 1e-5), D.RMS_NORM_F16_K_128_SMEM(1, 1e-6),
        D.RMS_NORM_F16_K_2048_SMEM(2, 1e-6), D.ROPE_INTERLEAVE_512(), D.SILU_MUL_SHARED_BF16_K_64_SW128(8),
        D.SILU_MUL_SHARED_BF16_K_4096_INTER(1), D.ARGMAX_PARTIAL_bf16_1024_65536_128(8), D.ARGMAX_REDUCE_bf16_1024_128(1),
    ])
    # ---------------------------------------------------------------- hardware loops
    ld = lambda: mi(op.OP_ALLOC_TMA_LOAD_1D, 1, 0, 8192, address=0x10000)
    st = lambda: mi(op.OP_ALLOC_WB_TMA_STORE_1D, 1, 0, 8192, address=0x90000)
    cases["repeat_on"] = encode(D.RepeatM.on(6, [ld(), 8192], [st(), 8192]) + D.RepeatM.on(1, [ld(), 64]) +
                                D.RepeatM.on(4, [ld(), 0x100], [ld(), 0x100], [st(), [0, 8, 0, 0]]))
    cases["repeat_on1_onsync"] = encode(D.RepeatM.on1(5, [ld(), 4096], [st(), 4096]) +
                                        D.RepeatM.onSync(0, 23, 4, [ld(), 8192], [ld(), 8192], [st(), 1024]) +
                                        D.RepeatM.onSync(1, 9, 3, [ld(), 8192], [ld(), 8192], asyncPort=False) +
                                        D.RepeatM.onSync(0, None, 3, [ld(), 8192]))
    return cases


def build_attention_cases(D, M):
    """Decode attention: the operator encodings, the strided tensor-map recipes of dae.model (M) and a
    SchedAttentionDecoding launch with the fused QK-norm + RoPE path (streams, barrier table, tensor maps)."""
    from functools import partial
    T = FakeTensor
    cases = {}
    cases["attention_compute"] = encode([
        D.ATTENTION_M64N64K16_F16_F32_64_64_hdim(3, 17), D.ATTENTION_M64N64K16_F16_F32_64_64_hdim_MMA(2, 64, False, False),
        D.ATTENTION_M64N64K16_F16_F32_64_64_hdim_split(2, 1, 4, 40, 128),
        D.ATTENTION_M64N64K16_F16_F32_64_64_hdim_split_MMA(5, 15, 8, 1, 4096), D.ATTN_SPLIT_POST_REDUCE(2),
    ])
    n_req, S, n_heads, Dh, blk = 2, 192, 8, 128, 64
    q, o = T((n_req, n_heads, 1, Dh)), T((n_req, n_heads, Dh), addr=0x7f08_0000_0000)
    k, v = T((n_req, S, n_heads, Dh), addr=0x7f10_0000_0000), T((n_req, S, n_heads, Dh), addr=0x7f18_0000_0000)
    side = T((S, 3 * Dh), addr=0x7f20_0000_0000)
    dae = D.Launcher(n_req * n_heads, device="cpu")
    tQ = D.TmaTensor(dae, q)._build("load", Dh, 64, M.tma_gqa_load_q, M.cord_gqa_load_q)
    tK = D.TmaTensor(dae, k)._build("load", Dh, blk, partial(M.build_tma_wgmma_k, iN=-3), partial(M.cord_func_K_major, iN=-3))
    tV = D.TmaTensor(dae, v)._build("load", Dh, blk, partial(M.build_tma_wgmma_mn, iK=-3), partial(M.cord_func_MN_major, iK=-3))
    tSide = D.TmaTensor(dae, side).tensor1d("load", 3 * Dh)
    kst = [D.TmaTensor(dae, T((S, n_heads * Dh), addr=0x7f10_0000_0000 + r * S * n_heads * Dh * 2)).tensor1d("store", Dh)
           for r in range(n_req)]
    g = dae.add_group("attn", 1)
    g.addBarrier("bar_q", 1)
    g.addBarrier("bar_k", 1)
    g.addBarrier("bar_o")                      # bound late, from the schedule's own count
    dae.build_groups()
    sched = D.SchedAttentionDecoding(n_req, 150, blk, n_heads, o, (tQ, tK, tV), side_input=tSide, k_store=kst, token_pos=149) \
        .bar("q", g["bar_q"]).bar("k", g["bar_k"]).bar("o", g["bar_o"]).place(n_req * n_heads)
    dae.bind_late_barrier_counts(sched)
    dae.s(sched)
    plain = D.SchedAttentionDecoding(n_req, 64, blk, n_heads, o, (tQ, tK, tV)).place(n_req * n_heads)
    dae.s(plain)
    dae.build_instructions()
    used_c, used_m = min(dae.cptrs), min(dae.mptrs)      # every SM has written at least this many (the rest of a ring is unspecified)
    cases["attention_cinsts"] = dae.cinsts[:, :used_c].numpy().copy().reshape(-1)
    cases["attention_minsts"] = dae.minsts[:, :used_m].numpy().copy().reshape(-1)
    cases["attention_bars"] = np.array([dae.bar_values[i] for i in range(dae.num_bars)], dtype=np.int64).view(np.uint8)
    cases["attention_tmas"] = torch.stack(dae.tmas).numpy().copy().reshape(-1)
    k2 = T((4, 256, 128), addr=0x7f30_0000_0000)
    recs = [M.build_tma_wgmma_k(k2, 128, 64)[1], M.build_tma_wgmma_mn(k2, 128, 64)[1], M.build_tma_wgmma_mn(k2, 64, 32)[1]]
    cases["model_recipes"] = torch.stack(recs).numpy().copy().reshape(-1)
    cords = [M.cord_func_K_major(k, 4, iN=-3)(1, 64, 3, 0), M.cord_func_MN_major(k, 5, iK=-3)(1, 128, 5, 64),
             M.cord_func_K_major(k2, 4)(2, 64, 64), M.cord_func_MN_major(k2, 5)(3, 16, 64),
             M.cord_func_MN_major_cord2(k2, 5)(16, 64), M.cord_gqa_load_q(q, 5)(1, 6), M.get_other_dims(4, -3)]
    cases["model_cords"] = np.array([c + [0] * (4 - len(c)) for c in cords], dtype=np.int64).reshape(-1).view(np.uint8)
    return cases


def build_launcher_cases(D):
    """A small two-projection "layer" replayed by device-side loops, built the way the reference's model
    scripts build theirs (app/python/llama3/sched.py:58-571): resource groups, late-bound barriers, tiled
    projections with split-K reduce stores, RMSNorm, SiLU on register tiles, argmax, LoopM / LoopC."""
    T = FakeTensor
    N, H, F, L, S = 8, 2048, 2048, 3, 32
    dae = D.Launcher(S, device="cpu")
    layerg = dae.add_group("layer", L)
    sysg = dae.add_group("system", 1)
    dae.get_group().addBarrier("bar_embedding", N)
    sysg.addBarrier("bar_val")
    sysg.addBarrier("bar_idx")
    sysg.addBarrier("bar_final")
    for name in ("bar_in", "bar_act", "bar_out"):
        layerg.addBarrier(name)
    layerg.addBarrier("bar_rms", N)
    Atom = D.Gemv_M64N8
    TileM, _, TileK = Atom.MNK
    hidden, act = T((N, H)), T((N, F), addr=0x7f10_0000_0000)
    ups = [T((F, H), addr=0x7f20_0000_0000 + l * F * H * 2) for l in range(L)]
    gates = [T((F, H), addr=0x7f28_0000_0000 + l * F * H * 2) for l in range(L)]
    downs = [T((H, F), addr=0x7f30_0000_0000 + l * F * H * 2) for l in range(L)]
    rmsw = [T((H,), addr=0x7f40_0000_0000 + l * H * 2) for l in range(L)]
    layerg.addTma("loadHidden", [hidden] * L, lambda t: t.wgmma_load(N, TileK * Atom.n_batch, D.Major.K))
    layerg.addTma("loadAct", [act] * L, lambda t: t.wgmma_load(N, TileK * Atom.n_batch, D.Major.K))
    layerg.addTma("storeAct", [act] * L, lambda t: t.wgmma_store(N, TileM, D.Major.MN))
    layerg.addTma("reduceHidden", [hidden] * L, lambda t: t.wgmma("reduce", N, TileM, D.Major.MN))
    layerg.addTma("loadUp", ups, lambda t: t.wgmma_load(TileM, TileK, D.Major.K))
    layerg.addTma("loadGate", gates, lambda t: t.wgmma_load(TileM, TileK, D.Major.K))
    layerg.addTma("loadDown", downs, lambda t: t.wgmma_load(TileM, TileK, D.Major.K))
    layerg.addTma("loadRmsW", rmsw, lambda t: t.tensor1d("load", H))
    dae.build_groups()
    g = layerg
    rms_io = D.TmaLoad1D(hidden, bytes=H * 2), D.TmaStore1D(hidden, bytes=H * 2)
    rms = D.SchedRMSShared(N, 1e-5, (g["loadRmsW"], *rms_io)).bar("input", g["bar_in"]).bar("output", g["bar_rms"]).place(8)
    up = D.SchedGemv(Atom, (F, N, H), (g["loadUp"], g["loadHidden"], D.RegStore(0, size=TileM * N * 2))) \
        .bar("load", g["bar_rms"]).place(F // TileM)
    gate = D.SchedGemv(Atom, (F, N, H), (g["loadGate"], g["loadHidden"], D.RegStore(1, size=TileM * N * 2))).place(F // TileM)
    silu = D.SchedRegSiLUFused(N, g["storeAct"], 1, 0, 0, TileM).bar("output", g["bar_act"]).place(F // TileM)
    down = D.SchedGemv(Atom, (H, N, F), (g["loadDown"], g["loadAct"], g["reduceHidden"]), fold=1) \
        .bar("load", g["bar_act"]).bar("store", g.next("bar_in")).place(H // TileM)
    down2 = D.SchedGemv(Atom, ((0, 512), N, F), (g["loadDown"], g["loadAct"], g["reduceHidden"]), fold=2) \
        .bar("store", g["bar_out"]).place(16)
    logits = [T((N, 1024), addr=0x7f50_0000_0000), T((N, 1024), addr=0x7f51_0000_0000)]
    oval, oidx, fin = T((N, S), addr=0x7f60_0000_0000), T((N, S), 8, addr=0x7f61_0000_0000), T((N,), 8, addr=0x7f62_0000_0000)

    class P(D.ARGMAX_PARTIAL_bf16_1024_65536_128):
        CHUNK_SIZE, I_STRIDE, SMS = 64, 1024, S

    class R(D.ARGMAX_REDUCE_bf16_1024_128):
        CHUNK_SIZE, SMS = 64, S
    argmax = D.SchedArgmax(N, 1024, 2, P, R, logits, oval, oidx, fin).bar("val", sysg["bar_val"]) \
        .bar("idx", sysg["bar_idx"]).bar("final", sysg["bar_final"]).place(S)
    layer = [rms, up, gate, silu, down, down2]
    dae.bind_late_barrier_counts(*layer, argmax)
    loop_m, loop_c = dae.copy_mptrs(), dae.copy_cptrs()
    dae.i(*layer, D.LoopM.toNext(loop_m, L, resource_group=layerg), D.LoopC.toNext(loop_c, L))
    dae.i(D.SchedCopy((D.ToLinearCordAdapter(D.TmaLoad1D(T((S, 64), 4)), 256),
                       D.ToLinearCordAdapter(D.TmaStore1D(T((S, 64), 4, addr=0x7f70_0000_0000)), 256))).place(S))
    dae.s(argmax)
    dae.build_instructions()
    cases = {}
    used_c = max(dae.cptrs) + 1
    used_m = max(dae.mptrs) + 1
    cases["launcher_cinsts"] = dae.cinsts[:, :used_c].numpy().copy().reshape(-1)
    cases["launcher_minsts"] = dae.minsts[:, :used_m].numpy().copy().reshape(-1)
    cases["launcher_bars"] = np.array([dae.bar_values[i] for i in range(dae.num_bars)], dtype=np.int64).view(np.uint8)
    cases["launcher_tmas"] = torch.stack(dae.tmas).numpy().copy().reshape(-1)
    cases["launcher_ptrs"] = np.array(dae.cptrs + dae.mptrs, dtype=np.int64).view(np.uint8)
    return cases
