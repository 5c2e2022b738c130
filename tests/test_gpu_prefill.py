"""Prefill on the device against the CPU oracle: the prompt's cache rows (every layer) within the hidden-state bar,
the first generated id equal wherever the oracle's top-2 logit gap exceeds 1e-2, and decode continuing from the
prefilled pools on the oracle's trajectory.  Two paths: a chunk of positions per launch (prefill.PrefillEngine)
and one position per launch through the decode program (DecodeEngine.prefill_device)."""
import pytest
import torch

from oracle import decode_oracle as O
from tests.helpers import dense_weights, engine_config, perturb_norms, small_cfg

pytestmark = pytest.mark.gpu
REL_L2_BF16 = 1e-2
GAP = 1e-2


def _setup(kind, prompt_len, cuda_device, seed, page_perm_seed=None):
    from vdcores_b200.decode import DecodeEngine
    cfg = small_cfg(kind)
    w = perturb_norms(O.ModelWeights.random(cfg, seed=seed))
    prompt = torch.randint(0, cfg.vocab, (prompt_len,), generator=torch.Generator().manual_seed(seed + 20))
    orc = O.DecodeOracle(w, 256)
    _, nxt, gap = orc.prefill(prompt.tolist())
    eng = DecodeEngine(engine_config(cfg), max_seq=256, device=cuda_device, timeout_ns=500_000_000,
                       page_perm_seed=page_perm_seed)
    eng.load_weights(dense_weights(w))
    return cfg, prompt, orc, nxt, gap, eng


def _check_cache_and_continue(cfg, T, orc, nxt, gap, eng, first, n_steps=4):
    for l in range(cfg.n_layers):
        k_dev, v_dev = eng.read_kv(l, T)
        # rows of layer l derive from the input of layer l: the hidden-state bar, doubled as in the decode test
        assert O.rel_l2(k_dev.cpu(), orc.k[l][:T]) < 2 * REL_L2_BF16, f"K rows of layer {l}"
        assert O.rel_l2(v_dev.cpu(), orc.v[l][:T]) < 2 * REL_L2_BF16, f"V rows of layer {l}"
        # and row by row: no position of a chunk may be off (a causal-mask or ordering slip shows in single rows)
        kd, ko = k_dev.cpu().float().flatten(1), orc.k[l][:T].float().flatten(1)
        assert float(((kd - ko).norm(dim=1) / ko.norm(dim=1)).max()) < 4 * REL_L2_BF16, f"a K row of layer {l}"
    if gap > GAP:
        assert first == nxt
    tok = nxt
    eng.set_state(T, tok)
    for _ in range(n_steps):
        _, ref_next, g = orc.step(tok)
        got = eng.step_host(tok)
        if g > GAP:
            assert got == ref_next
        tok = ref_next


@pytest.mark.parametrize("kind,prompt_len,chunk,perm", [("llama", 150, 16, None), ("llama", 129, 64, 7),
                                                        ("qwen3", 100, 32, 3), ("llama", 5, 16, None),
                                                        ("llama", 200, 128, 9), ("qwen3", 150, 128, None)])
def test_chunked_prefill_matches_oracle(cuda_device, kind, prompt_len, chunk, perm):
    """Chunks that end inside a page, a ragged last chunk, a prompt shorter than one chunk, shuffled page ids,
    per-head q/k norms; with 128 positions per launch there are more attention units than SMs and a unit walks
    its pages alone, two per trip (with and without two positions per unit)."""
    from vdcores_b200.prefill import PrefillEngine
    cfg, prompt, orc, nxt, gap, eng = _setup(kind, prompt_len, cuda_device, seed=21, page_perm_seed=perm)
    pre = PrefillEngine(eng, chunk=chunk, timeout_ns=500_000_000).adopt_weights()
    assert pre.kpool.data_ptr() == eng.kpool.data_ptr()           # the decode engine's own pools
    first = pre.prefill(prompt)
    _check_cache_and_continue(cfg, prompt_len, orc, nxt, gap, eng, first)


def test_chunked_prefill_agrees_with_the_pytorch_prefill(cuda_device):
    """Same prompt through the library-GEMM prefill and the megakernel prefill: same first id (outside near-ties),
    cache rows within the bf16 bar of each other."""
    from vdcores_b200.prefill import PrefillEngine
    cfg, prompt, orc, nxt, gap, eng = _setup("llama", 200, cuda_device, seed=23)
    first_torch = eng.prefill(prompt)
    ref = [[t.clone() for t in eng.read_kv(l, 200)] for l in range(cfg.n_layers)]
    eng.kpool.zero_()
    eng.vpool.zero_()
    first = PrefillEngine(eng, chunk=64, timeout_ns=500_000_000).adopt_weights().prefill(prompt)
    for l in range(cfg.n_layers):
        k_dev, v_dev = eng.read_kv(l, 200)
        assert O.rel_l2(k_dev, ref[l][0]) < 2 * REL_L2_BF16 and O.rel_l2(v_dev, ref[l][1]) < 2 * REL_L2_BF16
    if gap > GAP:
        assert first == first_torch == nxt


@pytest.mark.parametrize("kind,prompt_len", [("llama", 70), ("moe", 40)])
def test_position_by_position_prefill_matches_oracle(cuda_device, kind, prompt_len):
    """The decode program itself run over the prompt with forced ids (dense and mixture-of-experts models)."""
    cfg, prompt, orc, nxt, gap, eng = _setup(kind, prompt_len, cuda_device, seed=25)
    first = eng.prefill_device(prompt)
    _check_cache_and_continue(cfg, prompt_len, orc, nxt, gap, eng, first, n_steps=3)


@pytest.mark.parametrize("wkind,tol,base", [("fp8", 3e-2, "llama"), ("nvfp4", 6e-2, "qwen3_1k")])
def test_chunked_prefill_with_quantised_projections(cuda_device, wkind, tol, base):
    """The prefill engine adopts the decode engine's stored e4m3 / NVFP4 projections (same codes and scales,
    repacked for the tensor-core tasks); cache rows against the oracle that dequantises the same codes."""
    import copy
    import dataclasses
    from vdcores_b200.decode import DecodeEngine
    from vdcores_b200.prefill import PrefillEngine
    cfg_b = small_cfg(base)
    w_b = perturb_norms(O.ModelWeights.random(cfg_b, seed=6))
    cfg = dataclasses.replace(cfg_b, wkind=wkind)
    w = copy.copy(w_b)
    w.cfg = cfg
    w.layers = []
    for lw in w_b.layers:
        q = copy.copy(lw)
        for name in ("wq", "wk", "wv", "wo", "gate", "up", "down"):
            setattr(q, name, O.QLinear.make(getattr(lw, name).w, wkind))
        w.layers.append(q)
    T = 90
    prompt = torch.randint(0, cfg.vocab, (T,), generator=torch.Generator().manual_seed(31))
    orc = O.DecodeOracle(w, 128)
    _, nxt, gap = orc.prefill(prompt.tolist())
    eng = DecodeEngine(engine_config(cfg), max_seq=128, device=cuda_device, wkind=wkind, timeout_ns=500_000_000)
    eng.load_weights(dense_weights(w_b))
    first = PrefillEngine(eng, chunk=32, timeout_ns=500_000_000).adopt_weights().prefill(prompt)
    for l in range(cfg.n_layers):
        k_dev, v_dev = eng.read_kv(l, T)
        assert O.rel_l2(k_dev.cpu(), orc.k[l][:T]) < 2 * tol and O.rel_l2(v_dev.cpu(), orc.v[l][:T]) < 2 * tol
    if gap > 5 * GAP:
        assert first == nxt


def test_long_walks_agree_with_the_decode_program(cuda_device):
    """A 1000-token prompt, 128 positions per launch: units walk up to 16 pages two at a time, through every page
    count whose odd tail page once shared an arrival counter with the trip before it (15 pages: positions 896..959).
    Checked against the same prompt run position by position through the decode program (itself checked against the
    oracle above): cache rows of every layer, first generated id."""
    from vdcores_b200.decode import DecodeEngine
    from vdcores_b200.prefill import PrefillEngine
    cfg = small_cfg("llama")
    w = perturb_norms(O.ModelWeights.random(cfg, seed=27))
    T = 1000
    prompt = torch.randint(0, cfg.vocab, (T,), generator=torch.Generator().manual_seed(28))
    eng = DecodeEngine(engine_config(cfg), max_seq=1088, device=cuda_device, timeout_ns=500_000_000)
    eng.load_weights(dense_weights(w))
    first_ref = eng.prefill_device(prompt)
    ref = [[t.clone() for t in eng.read_kv(l, T)] for l in range(cfg.n_layers)]
    top2 = torch.topk(eng.logits.float(), 2).values
    eng.kpool.zero_()
    eng.vpool.zero_()
    pre = PrefillEngine(eng, chunk=128, timeout_ns=500_000_000).adopt_weights()
    assert pre.n_splits == 1 and pre.pages_per_split == 17
    first = pre.prefill(prompt)
    for l in range(cfg.n_layers):
        k_dev, v_dev = eng.read_kv(l, T)
        assert O.rel_l2(k_dev, ref[l][0]) < 2 * REL_L2_BF16 and O.rel_l2(v_dev, ref[l][1]) < 2 * REL_L2_BF16, f"layer {l}"
        kd, ko = k_dev.float().flatten(1), ref[l][0].float().flatten(1)
        assert float(((kd - ko).norm(dim=1) / ko.norm(dim=1)).max()) < 4 * REL_L2_BF16, f"a K row of layer {l}"
    if float((top2[0] - top2[1]) / top2[0].abs()) > 5 * GAP:
        assert first == first_ref
