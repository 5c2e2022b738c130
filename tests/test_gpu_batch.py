"""Batched decode on the tensor cores: operator-level checks of the tcgen05
projection task against an fp32 matmul, then end-to-end parity of the batched
engine with one CPU oracle per sequence (same bars as batch 1: per-layer hidden
states within rel-L2 1e-2, greedy tokens identical where the oracle's top-2
logit gap exceeds 1e-2)."""
import pytest
import torch

from oracle import decode_oracle as O
from tests.helpers import dense_weights, engine_config, perturb_norms, small_cfg
from tests.test_gpu_ops import run_program, seeded

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
REL_L2_BF16 = 1e-2
GAP = 1e-2


def _bpad(B):
    return next(p for p in (16, 32, 64, 128) if B <= p)


def _gemm_program(dev, x, w, n_sms, mode, out, norm_w=None, eps=1e-5, ld=0, keys=None, stats=None, scales=None,
                  wfmt=None, n_rows=None):
    """w: bf16 weights, or (with scales) uint8 e4m3 codes / NVFP4 rows (wfmt "nvfp4") and their fp32 per-row scales."""
    from vdcores_b200.batch import (BLOCK_ROWS, emit_projection, pack_blocks, pack_blocks_fp8, pack_blocks_nvfp4, pack_kc,
                                    projection_blocks)
    from vdcores_b200.program import Program
    B, K = x.shape
    Bp = _bpad(B)
    xp = torch.zeros(Bp, K, dtype=BF16)
    xp[:B] = x
    xd = pack_kc(xp.to(dev))
    wfmt = wfmt or ("fp8" if scales is not None else "bf16")
    wd = {"fp8": pack_blocks_fp8, "bf16": pack_blocks, "nvfp4": lambda t: pack_blocks_nvfp4(t, K)}[wfmt](w.to(dev))
    sd = scales.to(dev) if scales is not None else None
    nwd = norm_w.to(dev) if norm_w is not None else None
    if norm_w is not None:      # the producers of a normed input leave its per-row sums of squares
        stats = torch.zeros(128, dtype=torch.float32)
        stats[:B] = x.float().pow(2).sum(-1)
        stats = stats.to(dev)
    n_blocks = len(projection_blocks(w.shape[0]))
    scr = torch.zeros(n_blocks * B * BLOCK_ROWS, dtype=torch.float32, device=dev)
    cnt = torch.zeros(n_blocks, dtype=torch.int32, device=dev)
    P = Program(n_sms)
    units = emit_projection(P, sms=list(range(n_sms)), load=[0] * n_sms, w_addr=wd.data_ptr(), M=w.shape[0], K=K,
                            x_addr=xd.data_ptr(), B=B, Bpad=Bp, mode=mode, out_addr=out.data_ptr() if out is not None else 0,
                            scratch_addr=scr.data_ptr(), counter_addr=cnt.data_ptr(),
                            norm_addr=nwd.data_ptr() if nwd is not None else None, eps=eps, ld=ld,
                            keys_addr=keys.data_ptr() if keys is not None else 0,
                            stats_addr=stats.data_ptr() if stats is not None else 0,
                            wfmt=wfmt, scales_addr=sd.data_ptr() if sd is not None else 0)
    run_program(P, dev)
    assert float(scr.abs().max()) == 0.0 and int(cnt.abs().max()) == 0, "scratch and counters are left clear"
    return units


@pytest.mark.parametrize("B,K,M,n_sms,norm", [(5, 512, 96, 2, False), (16, 4096, 640, 5, True),
                                             (40, 1024, 256, 1, True), (100, 256, 64, 3, False),
                                             (16, 14336, 512, 7, False)])
def test_gemm_tc_store_rows(cuda_device, B, K, M, n_sms, norm):
    from vdcores_b200 import isa
    dev = cuda_device
    x, w = seeded((B, K), 21), seeded((M, K), 22, 0.05)
    nw = (1 + 0.1 * torch.randn(K, generator=torch.Generator().manual_seed(23))).to(BF16) if norm else None
    y = torch.zeros(B, M, dtype=BF16, device=dev)
    units = _gemm_program(dev, x, w, n_sms, isa.GEMM_MODE_STORE_ROWS, y, norm_w=nw, ld=M)
    if n_sms > 1:
        assert len(units) > len({u[1] for u in units}), "some block's K is shared by several units"
    xin = O.rms_norm(x, nw, 1e-5) if norm else x
    ref = O.linear(xin, w)
    assert O.rel_l2(y.cpu(), ref) < 4e-3


@pytest.mark.parametrize("B,K,M,n_sms,norm", [(7, 512, 256, 1, False), (16, 4096, 640, 5, True), (40, 1024, 96, 2, False)])
def test_gemm_tc_fp8_weights(cuda_device, B, K, M, n_sms, norm):
    """e4m3 weights with per-row scales: converted to bf16 in shared memory, scaled in the epilogue;
    compared with the oracle's linear layer over the same codes."""
    from vdcores_b200 import isa
    from vdcores_b200.decode import quantize_fp8_rows
    dev = cuda_device
    x, w = seeded((B, K), 41), seeded((M, K), 42, 0.05)
    codes, scales = quantize_fp8_rows(w)
    nw = (1 + 0.1 * torch.randn(K, generator=torch.Generator().manual_seed(43))).to(BF16) if norm else None
    y = torch.zeros(B, M, dtype=BF16, device=dev)
    _gemm_program(dev, x, codes, n_sms, isa.GEMM_MODE_STORE_ROWS, y, norm_w=nw, ld=M, scales=scales)
    wq = (codes.view(torch.float8_e4m3fn).float() * scales[:, None])
    xin = O.rms_norm(x, nw, 1e-5) if norm else x
    ref = (xin.float() @ wq.t()).to(BF16)
    assert O.rel_l2(y.cpu(), ref) < 4e-3


@pytest.mark.parametrize("B,K,M,n_sms,norm", [(7, 512, 256, 1, False), (16, 4096, 640, 5, True), (40, 1024, 96, 2, False)])
def test_gemm_tc_nvfp4_weights(cuda_device, B, K, M, n_sms, norm):
    """NVFP4 weights (e2m1 values, one e4m3 scale per 16 inputs, fp32 tensor scale): value times block scale is
    converted to bf16 in shared memory (exact), the tensor scale applied in the epilogue; compared with the
    oracle's linear layer over the same codes."""
    from vdcores_b200 import isa
    dev = cuda_device
    x, w = seeded((B, K), 51), seeded((M, K), 52, 0.05)
    from vdcores_b200.decode import quantize_nvfp4_rows
    lin = O.QLinear.make(w, "nvfp4")
    rows, ts = quantize_nvfp4_rows(w)          # the engine's codec: the same codes as the oracle's
    assert torch.equal(rows[:, :K // 2], lin.q)
    scales = ts.expand(M).contiguous()
    nw = (1 + 0.1 * torch.randn(K, generator=torch.Generator().manual_seed(53))).to(BF16) if norm else None
    y = torch.zeros(B, M, dtype=BF16, device=dev)
    _gemm_program(dev, x, rows, n_sms, isa.GEMM_MODE_STORE_ROWS, y, norm_w=nw, ld=M, scales=scales, wfmt="nvfp4")
    xin = O.rms_norm(x, nw, 1e-5) if norm else x
    assert O.rel_l2(y.cpu(), lin(xin)) < 4e-3


def test_gemm_tc_residual_add_and_silu(cuda_device):
    from vdcores_b200 import isa
    from vdcores_b200.batch import pack_kc, unpack_kc
    dev = cuda_device
    B, K, M = 12, 768, 512
    Bp = 16
    x, w = seeded((B, K), 24), seeded((M, K), 25, 0.05)
    h0 = seeded((B, M), 26)
    hp = torch.zeros(Bp, M, dtype=BF16)
    hp[:B] = h0
    hd = pack_kc(hp.to(dev))
    stats = torch.zeros(128, dtype=torch.float32, device=dev)
    _gemm_program(dev, x, w, 3, isa.GEMM_MODE_ADD_PACKED, hd, stats=stats)
    got = unpack_kc(hd, Bp, M)[:B].cpu()
    ref = (h0.float() + O.linear(x, w).float()).to(BF16)
    assert O.rel_l2(got, ref) < 4e-3
    # the task also leaves the updated rows' sums of squares for the next RMSNorm
    assert torch.allclose(stats[:B].cpu(), got.float().pow(2).sum(-1), rtol=1e-4)
    assert float(stats[B:].abs().max()) == 0.0
    assert float(unpack_kc(hd, Bp, M)[B:].float().abs().max()) == 0.0   # padding rows stay untouched

    F = 256
    gate, up = seeded((F, K), 27, 0.05), seeded((F, K), 28, 0.05)
    wgu = torch.stack((gate, up), dim=1).reshape(2 * F, K).contiguous()
    ad = torch.zeros(Bp * F, dtype=BF16, device=dev)
    _gemm_program(dev, x, wgu, 2, isa.GEMM_MODE_SILU_PAIRS, ad)
    got = unpack_kc(ad, Bp, F)[:B].cpu()
    ref = O.silu_mul(O.linear(x, gate), O.linear(x, up))
    assert O.rel_l2(got, ref) < 5e-3


def test_gemm_tc_argmax_keys(cuda_device):
    from vdcores_b200 import isa
    dev = cuda_device
    B, K, V = 9, 512, 2048
    x, w = seeded((B, K), 29), seeded((V, K), 30, 0.05)
    w[1500] = w[300]        # identical logits in two rows: the lower id must win when they are the maximum
    x[0] = (w[300].float() * 50).to(BF16)
    keys = torch.zeros(B, dtype=torch.int64, device=dev)
    _gemm_program(dev, x, w, 4, isa.GEMM_MODE_ARGMAX, None, keys=keys)
    low = (keys.cpu() & 0xFFFFFFFF).tolist()
    got = [0xFFFFFFFF - v for v in low]
    ref = O.linear(x, w).float()
    assert got[0] == 300
    for b in range(B):
        assert float(ref[b, got[b]]) >= float(ref[b].max()) - 1e-2 * float(ref[b].abs().max())


@pytest.mark.parametrize("kind,batch,num_sms", [("llama", 3, None), ("qwen3", 20, None), ("llama", 20, 32)])
def test_batch_decode_matches_oracle(cuda_device, kind, batch, num_sms):
    """20 sequences x 2 KV heads on 32 SMs: more attention units than SMs, so a unit walks all four pages of its
    sequence alone, two pages per trip (contexts of 4, 3 and 2 pages: last page second in a trip, odd tail page,
    single trip)."""
    from vdcores_b200.batch import BatchDecodeEngine
    cfg = small_cfg(kind)
    w = perturb_norms(O.ModelWeights.random(cfg, seed=3))
    g = torch.Generator().manual_seed(31)
    lens = [int(v) for v in torch.randint(2, 150, (batch,), generator=g)]
    if batch > 4:       # the oracle prefill is the slow part: keep most prompts short
        lens = [l if b < 3 else 2 + l % 20 for b, l in enumerate(lens)]
    if num_sms is not None:
        lens[:3] = [200, 131, 100]
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g) for n in lens]
    eng = BatchDecodeEngine(engine_config(cfg), batch, max_seq=256, device=cuda_device, taps=True, page_perm_seed=5,
                            timeout_ns=500_000_000, num_sms=num_sms)
    assert num_sms is None or (eng.n_splits == 1 and eng.pages_per_split == 4)
    eng.load_weights(dense_weights(w))
    orcs, toks = [], []
    for b in range(batch):
        orc = O.DecodeOracle(w, 256)
        orc.prefill(prompts[b][:-1].tolist())
        n = lens[b] - 1
        eng.load_kv([k[:n] for k in orc.k], [v[:n] for v in orc.v], b=b)
        eng.set_state(n, int(prompts[b][-1]), b=b)
        orcs.append(orc)
        toks.append(int(prompts[b][-1]))
    for step in range(3):
        got = eng.generate(1)[0]
        taps = [eng.read_hidden(eng.taps[l]).cpu() for l in range(cfg.n_layers)]
        fix = {}
        for b in range(batch):
            caps = []
            _, nxt_ref, gap = orcs[b].step(toks[b], caps)
            for l in range(cfg.n_layers):
                r = O.rel_l2(taps[l][b], caps[l]["hidden_state_out"])
                assert r < REL_L2_BF16, f"step {step} sequence {b} layer {l}: rel-L2 {r:.3e}"
            if gap > GAP:
                assert got[b] == nxt_ref, f"step {step} sequence {b}: token {got[b]} vs {nxt_ref} (gap {gap:.3f})"
            if got[b] != nxt_ref:
                fix[b] = nxt_ref
            toks[b] = nxt_ref
            pos = lens[b] - 1 + step
            k_dev, v_dev = eng.read_kv(cfg.n_layers - 1, pos + 1, b=b)
            assert O.rel_l2(k_dev[pos].cpu(), orcs[b].k[-1][pos]) < 2 * REL_L2_BF16
            assert O.rel_l2(v_dev[pos].cpu(), orcs[b].v[-1][pos]) < 2 * REL_L2_BF16
        for b, t in fix.items():    # keep every sequence on its oracle's trajectory
            eng.state[b, 2:3].copy_(torch.tensor([t], dtype=torch.int32))


def test_batch_prefill_and_host_steps(cuda_device):
    """PyTorch prefill per sequence, then steps driven from host buffers follow the oracles."""
    from vdcores_b200.batch import BatchDecodeEngine
    cfg = small_cfg("llama")
    w = O.ModelWeights.random(cfg, seed=4)
    g = torch.Generator().manual_seed(32)
    batch, T = 4, 40
    prompts = torch.randint(0, cfg.vocab, (batch, T), generator=g)
    eng = BatchDecodeEngine(engine_config(cfg), batch, max_seq=128, device=cuda_device, timeout_ns=500_000_000)
    eng.load_weights(dense_weights(w))
    first = eng.prefill(prompts)
    orcs, toks = [], []
    for b in range(batch):
        orc = O.DecodeOracle(w, 128)
        _, nxt, gap = orc.prefill(prompts[b].tolist())
        if gap > GAP:
            assert first[b] == nxt
        orcs.append(orc)
        toks.append(nxt)
        eng.set_state(T, nxt, b=b)
    for _ in range(4):
        got = eng.step_host(toks)
        for b in range(batch):
            _, ref_next, gap = orcs[b].step(toks[b])
            if gap > GAP:
                assert got[b] == ref_next
            toks[b] = ref_next


@pytest.mark.parametrize("wkind,tol", [("fp8", 3e-2), ("nvfp4", 6e-2)])
def test_batch_decode_quantised_matches_oracle(cuda_device, wkind, tol):
    """Batched decode with e4m3 / NVFP4 layer projections against one oracle per sequence that dequantises
    the same codes: per-layer hidden states within rel-L2 3e-2 / 6e-2."""
    import copy
    import dataclasses
    from vdcores_b200.batch import BatchDecodeEngine
    cfg_b = small_cfg("llama")
    w_b = perturb_norms(O.ModelWeights.random(cfg_b, seed=6))
    cfg = dataclasses.replace(cfg_b, wkind=wkind)
    w = copy.copy(w_b)
    w.cfg = cfg
    w.layers = []
    for lw in w_b.layers:
        ql = copy.copy(lw)
        for name in ("wq", "wk", "wv", "wo", "gate", "up", "down"):
            setattr(ql, name, O.QLinear.make(getattr(lw, name).w, wkind))
        w.layers.append(ql)
    batch = 5
    g = torch.Generator().manual_seed(33)
    lens = [int(v) for v in torch.randint(2, 60, (batch,), generator=g)]
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g) for n in lens]
    eng = BatchDecodeEngine(engine_config(cfg), batch, max_seq=128, device=cuda_device, taps=True, wkind=wkind,
                            timeout_ns=500_000_000)
    eng.load_weights(dense_weights(w_b))       # the engine quantises the same bf16 weights with the same rule
    orcs, toks = [], []
    for b in range(batch):
        orc = O.DecodeOracle(w, 128)
        orc.prefill(prompts[b][:-1].tolist())
        n = lens[b] - 1
        eng.load_kv([k[:n] for k in orc.k], [v[:n] for v in orc.v], b=b)
        eng.set_state(n, int(prompts[b][-1]), b=b)
        orcs.append(orc)
        toks.append(int(prompts[b][-1]))
    for step in range(3):
        got = eng.generate(1)[0]
        taps = [eng.read_hidden(eng.taps[l]).cpu() for l in range(cfg.n_layers)]
        fix = {}
        for b in range(batch):
            caps = []
            _, nxt_ref, gap = orcs[b].step(toks[b], caps)
            for l in range(cfg.n_layers):
                r = O.rel_l2(taps[l][b], caps[l]["hidden_state_out"])
                assert r < tol, f"step {step} sequence {b} layer {l}: rel-L2 {r:.3e}"
            if gap > GAP:
                assert got[b] == nxt_ref
            if got[b] != nxt_ref:
                fix[b] = nxt_ref
            toks[b] = nxt_ref
        for b, t in fix.items():
            eng.state[b, 2:3].copy_(torch.tensor([t], dtype=torch.int32))
