"""A Hugging Face checkpoint directory straight into the engines, checked against the Hugging Face model itself:
tiny random LlamaForCausalLM / Qwen3ForCausalLM saved with save_pretrained, read by vdcores_b200.checkpoint, the
prompt prefilled through the megakernel, then greedy decode; logits within the bf16 bar of the Hugging Face forward
(bf16 on the host CPU), ids equal wherever its two best logits are more than a near-tie apart."""
import pytest
import torch

pytestmark = pytest.mark.gpu
REL_L2 = 2e-2       # logits after all layers, two bf16 implementations
GAP = 2e-2


def rel_l2(a, b):
    a, b = a.float().flatten(), b.float().flatten()
    return float((a - b).norm() / b.norm())


@pytest.mark.parametrize("family", ["llama", "qwen3"])
def test_checkpoint_to_prefill_to_decode_follows_hugging_face(cuda_device, tmp_path, family):
    tr = pytest.importorskip("transformers")
    from vdcores_b200 import checkpoint
    from vdcores_b200.decode import DecodeEngine
    from vdcores_b200.prefill import PrefillEngine
    kw = dict(hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
              num_key_value_heads=1, head_dim=128, vocab_size=2048, tie_word_embeddings=False,
              max_position_embeddings=512)
    torch.manual_seed(3)
    if family == "llama":
        model = tr.LlamaForCausalLM(tr.LlamaConfig(rms_norm_eps=1e-5, rope_theta=500000.0, **kw))
    else:
        model = tr.Qwen3ForCausalLM(tr.Qwen3Config(rms_norm_eps=1e-6, rope_theta=1000000.0, **kw))
    model = model.to(torch.bfloat16).eval()
    with torch.no_grad():                      # norm weights are 1 at init: move them so the affine part counts
        for n, p in model.named_parameters():
            if "norm" in n:
                p.mul_(1.0 + 0.1 * torch.randn(p.shape)).to(torch.bfloat16)
    model.save_pretrained(str(tmp_path), safe_serialization=True)

    cfg = checkpoint.read_config(str(tmp_path))
    eng = DecodeEngine(cfg, max_seq=256, device=cuda_device, timeout_ns=500_000_000)
    eng.load_weights(checkpoint.read_weights(str(tmp_path), cfg))
    T = 70
    ids = torch.randint(0, cfg.vocab, (T,), generator=torch.Generator().manual_seed(5))

    def hf_next(seq):
        with torch.no_grad():
            lg = model(torch.tensor([seq])).logits[0, -1].float()
        top2 = torch.topk(lg, 2).values
        return lg, int(torch.argmax(lg)), float((top2[0] - top2[1]) / top2[0].abs().clamp_min(1e-6))

    seq = ids.tolist()
    lg, nxt, gap = hf_next(seq)
    first = PrefillEngine(eng, chunk=32, timeout_ns=500_000_000).adopt_weights().prefill(ids)
    if gap > GAP:
        assert first == nxt
    tok = nxt
    eng.set_state(T, tok)
    for step in range(4):
        seq.append(tok)
        lg, nxt, gap = hf_next(seq)
        got = eng.step_host(tok)
        r = rel_l2(eng.logits.cpu(), lg)
        assert r < REL_L2, f"step {step}: logits rel-L2 {r:.3e} against Hugging Face"
        if gap > GAP:
            assert got == nxt, f"step {step}: {got} vs {nxt} (relative gap {gap:.3f})"
        tok = nxt
