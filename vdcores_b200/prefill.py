"""Prefill on the device: a chunk of consecutive prompt positions per launch of the megakernel.

The batched decode program (batch.BatchDecodeEngine: projections on the tensor cores, one attention unit per
(row, KV head)) already computes, for every row of its batch, exactly what a prompt position needs; what differs
in a prefill is that the rows are consecutive positions of ONE sequence.  PrefillEngine therefore gives every row
the same page table and position pos0 + b, and adds one stage per layer in front of the attention: cache-append
tasks (isa.ATTN_APPEND_BIT) write the normed, rotated key rows and the value rows of all the chunk's positions to
the paged pools; the attention units start behind that stage's barrier (their page copies are held back by the
same barrier), so position p finds the rows of every position < p of its own chunk in HBM, and its row limit
(pos + 1 rows of the last page) is the causal mask.  The pools and the page table are those of the decode engine
the prompt is prefilled for: nothing is copied when decode takes over.

The reference has no prefill of its own on the device either side of its decode schedules: its correctness runs
take the prompt's cache from a HuggingFace forward (app/python/llama3/sched.py:574-622 in the reference); this
engine replaces the PyTorch prefill of decode.DecodeEngine.prefill on the product path."""
import torch

from . import isa, runtime
from .batch import BatchDecodeEngine
from .decode import DecodeEngine


class PrefillEngine(BatchDecodeEngine):
    """`chunk` prompt positions per launch into the KV pools of `target` (a DecodeEngine of the same model)."""
    SHARED_CACHE = True

    def __init__(self, target: DecodeEngine, chunk: int = 64, timeout_ns: int = 2_000_000_000):
        assert not isinstance(target, BatchDecodeEngine) and not target.cfg.n_experts
        self.target = target
        super().__init__(target.cfg, chunk, target.max_seq, device=target.dev, num_sms=target.num_sms,
                         max_steps=1, timeout_ns=timeout_ns, wkind=target.wkind)
        self.rope = target.rope

    def _alloc_cache(self, page_perm_seed):
        t = self.target
        self.kpool, self.vpool = t.kpool, t.vpool
        self.page_table = t.page_table
        self.page_tables = t.page_table[None, :].expand(self.batch, -1).contiguous()

    def adopt_weights(self):
        """Takes the target's tensors (embedding, norms, vocabulary projection, the layer projections in their
        stored form: bf16 rows, e4m3 codes or NVFP4 rows, with their scales) and packs the projections for the
        tensor-core tasks; both engines store a projection the same way, only the packing differs."""
        t = self.target
        for name in ("embed", "lm_head", "norm_w", "ln1", "ln2", "qknorm", "wqkv", "wo", "wgu", "wd"):
            setattr(self, name, getattr(t, name))
        self.router, self.scales, self.w = None, dict(t.scales), True
        self._pack_cache = None
        self._build_program()
        return self

    def _build_program(self):
        """Two programs over the same packed weights: chunks before the prompt's last end after the last layer,
        the last chunk adds the final norm, the vocabulary projection and the argmax (the first generated id)."""
        self.WITH_VOCAB_PROJECTION = False
        super()._build_program()
        self._body = (self.insts_per_sm, self.cinsts, self.minsts, self.bars_init)
        self.WITH_VOCAB_PROJECTION = True
        super()._build_program()
        self._last = (self.insts_per_sm, self.cinsts, self.minsts, self.bars_init)

    # ------------------------------------------------------------------ chunks
    def _chunk_states(self, tokens: torch.Tensor) -> torch.Tensor:
        """State blocks [n_chunks, chunk, state_words] of a prompt: row b of chunk c is position c * chunk + b
        (rows past the prompt's end repeat its last position: same row, same bytes)."""
        T, B = int(tokens.numel()), self.batch
        n_chunks = (T + B - 1) // B
        pos = torch.arange(n_chunks * B).clamp_(max=T - 1)
        table = self.page_table.to(torch.int64)
        s = torch.zeros(n_chunks * B, self.state_words, dtype=torch.int32)
        s[:, isa.ST_POS] = pos.to(torch.int32)
        s[:, isa.ST_NPAGES] = (pos // isa.KV_PAGE + 1).to(torch.int32)
        s[:, isa.ST_TOKEN] = tokens.to(torch.int32)[pos]
        s[:, isa.ST_NEWROW] = (table[pos // isa.KV_PAGE] * isa.KV_PAGE * self.cfg.n_kv_heads + pos % isa.KV_PAGE).to(torch.int32)
        s[:, isa.ST_NKVH] = self.cfg.n_kv_heads
        s[:, isa.ST_MAXPAGES] = self.max_pages
        s[:, isa.ST_PAGETABLE:] = self.page_table
        return s.view(n_chunks, B, self.state_words)

    @torch.no_grad()
    def prefill(self, tokens: torch.Tensor, set_target_state: bool = True) -> int:
        """Runs the prompt, ceil(T / chunk) launches, and returns the first generated (greedy) id.  The only host
        work inside the loop is enqueueing, per chunk, the copy of its prepared state blocks and the launch."""
        T, B = int(tokens.numel()), self.batch
        assert 1 <= T < self.max_seq and self.program is not None
        states = self._chunk_states(tokens.cpu()).to(self.dev)
        self.attn_cnt.zero_()
        self.keys.zero_()
        self.stats.zero_()
        with torch.cuda.stream(self.stream):
            n = states.shape[0]
            for c in range(n):
                self.state.copy_(states[c], non_blocking=True)
                insts_per_sm, cinsts, minsts, bars_init = self._last if c == n - 1 else self._body
                runtime.launch_async(self.num_sms, insts_per_sm, cinsts, minsts, None, self.bars, bars_init,
                                     self.profile, self.stream.cuda_stream, self.timeout_ns, full=True)
        runtime.read_status(self.stream.cuda_stream)
        first = int(self.token_log[(T - 1) % B, 0])
        if set_target_state:
            self.target.set_state(T, first)
        return first
