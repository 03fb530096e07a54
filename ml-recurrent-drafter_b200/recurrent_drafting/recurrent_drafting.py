"""The ReDrafter decode loop on the B200 kernels, with the reference's interface
(recurrent_drafting/recurrent_drafting.py): RecurrentDrafting(llm, drafter).generate(ledger,
input_ids, max_length, beam_shape, sampling_args, special_tokens) yields the (batch, <= max_length)
int64 token matrix after every step.

One step enqueues, without reading anything back:
  drafter beam search -> prefix-tree pack (flat rows, cache slots, RoPE positions, bitmask)
  -> Llama verify forward over the packed tokens (K/V written straight into the cache)
  -> LM head -> argmax (greedy) or sparse top-50 log-softmax (sampling)
  -> acceptance + commit of the accepted path's tokens, K/V rows and next-step inputs.
Then one small device->host copy (row lengths, accepted counts) sizes the yielded tensor.

Cache rows never move and are stored left-compacted: the first real token of row b sits in slot
kv_begin[b] = 0 whatever the prompt's left padding, and the row only grows (kv_len[b]).  The furthest
slot a step can write is therefore max_b kv_len[b] + W*Lb, which the reference's allocation
(max_length + W*Lb) always covers.  The reference re-right-aligns every row after each step; its
slot numbering is available in index space through reference_commit_slots().
"""
import contextlib
import os
from dataclasses import dataclass
from typing import Generator, Optional, Tuple

import torch

from . import _lib, kv_cache, modeling_drafter, modeling_llama, stats, tree_attention


@dataclass
class SamplingArgs:
    temperature: float
    greedy: bool


@dataclass
class SpecialTokens:
    pad: int
    eos: Optional[int] = 1


def _count_left_paddings(tokens: torch.Tensor, pad_token_id: int) -> torch.Tensor:
    """Number of leading pad ids of every row (recurrent_drafting.py:387-388)."""
    return torch.sum(torch.cumprod(torch.eq(tokens, pad_token_id).to(torch.int64), dim=-1), dim=-1)


def _greedy_choose_from_candidates(beams_by_drafter: torch.Tensor, beams_by_llm: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """(n_tokens_in_seq, seq_in_beam) for per-beam (unpacked) LLM tokens (recurrent_drafting.py:468-496).
    Runs the acceptance kernel with an identity unpacker and no cache."""
    B, W, Lb = beams_by_drafter.shape
    dev = beams_by_drafter.device
    beams = beams_by_drafter.to(torch.int64).contiguous()
    llm_tok = beams_by_llm.to(torch.int32).reshape(-1).contiguous()
    unpacker = torch.arange(W * Lb, dtype=torch.int32, device=dev).repeat(B).contiguous()
    row_start = torch.arange(B + 1, dtype=torch.int32, device=dev) * (W * Lb)
    n = torch.empty(B, dtype=torch.int32, device=dev)
    seq = torch.empty(B, dtype=torch.int32, device=dev)
    nxt = torch.empty(B, dtype=torch.int64, device=dev)
    _lib.call("rd_accept_commit_greedy", _lib.F32, _lib.ptr(beams), B, W, Lb, _lib.ptr(unpacker), _lib.ptr(row_start),
              _lib.ptr(llm_tok), None, 0, None, 0, 0, 0, 0, None, None, None, None, _lib.ptr(n), _lib.ptr(seq), _lib.ptr(nxt),
              None, _lib.stream())
    return n.long(), seq.long()


class _DecodeState:
    """Device buffers of one generate() call."""

    def __init__(self, llm, B: int, W: int, Lb: int, max_len: int, device):
        H = llm.config.hidden_size
        i32 = dict(dtype=torch.int32, device=device)
        self.kv_begin = torch.zeros(B, **i32)
        # row 0: kv_len, row 1: n_accepted, row 2 [0]: status word of the tensor-core kernels (one read-back per step)
        self.small = torch.zeros(3, B, **i32)
        self.kv_len = self.small[0]
        self.n_accepted = self.small[1]
        self.small_host = torch.zeros(3, B, dtype=torch.int32).pin_memory()
        self.seq_in_beam = torch.zeros(B, **i32)
        self.token_buf = torch.zeros(B, max_len, dtype=torch.int64, device=device)
        self.ctx = torch.zeros(B, H, dtype=llm.dtype, device=device)
        self.init_tok = torch.zeros(B, dtype=torch.int64, device=device)
        self.llm_tok = torch.zeros(B * W * Lb, **i32)
        self.fp = tree_attention.alloc_flat(B, W, Lb, device)
        self.p = modeling_drafter.new_sparse(B * W * Lb, device)
        self.status = self.small[2, :1]
        # the uniforms of a sampling step: one per drafted position and one for the token after the accepted prefix
        self.u = torch.zeros(B, W, Lb - 1, dtype=torch.float32, device=device)
        self.u_next = torch.zeros(B, dtype=torch.float32, device=device)

    def draw_uniforms(self, B: int, W: int, Lb: int) -> None:
        """Fills u and u_next from torch's generator, in this order (the order the reference draws them in)."""
        for buf, shape in ((self.u, (B, W, Lb - 1)), (self.u_next, (B,))):
            r = torch.rand(*shape, device=buf.device, out=buf)
            if r is not buf:  # a stand-in for torch.rand that returns its own tensor
                buf.copy_(r)


class _StepGraphs:
    """The three phases of a decode step (draft, verify, accept) captured as CUDA graphs for one generate() call:
    a step is then three graph launches instead of some 260 kernel launches, which is what bounds small batches
    (the host needs 3-4 ms to enqueue a 7B step, a batch of one or two rows keeps the GPU busy for about as long).
    Captured after the first eager steps, when every TMA descriptor set and workspace exists; all tensors the
    phases touch live as long as the call, and nothing in them depends on a host value that changes per step."""

    def __init__(self):
        self.draft = self.verify = self.accept = None
        self.ready = False
        self.n_kernels = 0  # kernels captured in the three graphs together

    def capture(self, model: "RecurrentDrafting", st: _DecodeState, cache: kv_cache.Cache, beam_shape,
                sampling_args: "SamplingArgs") -> None:
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        graphs = [torch.cuda.CUDAGraph() for _ in range(3)]
        before = _lib.launches
        # Captured with capture_begin / capture_end rather than the torch.cuda.graph context manager: that one
        # synchronises the device and empties the allocator's caches (device and pinned host) before every capture,
        # after which the request's next allocations go back to cudaMalloc; the phases allocate nothing, so there is
        # nothing to make room for.  Three captures take 4-25 ms this way.  Thread-local capture mode: other threads of the process (a server's other requests) may keep calling
        # CUDA.
        def captured(graph, fn):
            graph.capture_begin(capture_error_mode="thread_local")
            try:
                return fn()
            finally:
                graph.capture_end()

        with torch.cuda.stream(stream):
            draft = captured(graphs[0], lambda: model._draft_phase(st, beam_shape))
            verified = captured(graphs[1], lambda: model._verify_phase(st, cache, beam_shape, sampling_args, draft, 0))
            captured(graphs[2], lambda: model._accept_phase(st, cache, beam_shape, sampling_args, draft, verified))
        torch.cuda.current_stream().wait_stream(stream)
        # capturing enqueues nothing: the calls made above are the kernels of every later replay
        self.n_kernels = _lib.launches - before
        _lib.launches = before
        self.draft, self.verify, self.accept = graphs
        self.ready = True


class RecurrentDrafting(torch.nn.Module):
    def __init__(self, llm: modeling_llama.LlamaForCausalLM, drafter: modeling_drafter.Drafter,
                 cuda_graphs: Optional[bool] = None):
        super().__init__()
        self.llm = llm
        self.drafter = drafter
        # replay each phase of a decode step from a CUDA graph (bf16, head_dim 128); the environment
        # variable RD_CUDA_GRAPHS=0/1 sets the default
        self.cuda_graphs = (os.environ.get("RD_CUDA_GRAPHS", "1") != "0") if cuda_graphs is None else bool(cuda_graphs)
        self.last_state: Optional[_DecodeState] = None
        self.last_cache: Optional[kv_cache.Cache] = None

    def llm_n_kv_heads(self) -> int:
        if isinstance(self.llm, modeling_llama.LlamaForCausalLM):
            return self.llm.n_kv_heads
        raise TypeError(f"Unsupported base model type {type(self.llm)}")

    def generate(self, ledger: stats.Ledger, input_ids: torch.Tensor, max_length: int,
                 beam_shape: modeling_drafter.BeamShape = modeling_drafter.BeamShape(10, -1),
                 sampling_args: SamplingArgs = SamplingArgs(1.0, False),
                 special_tokens: SpecialTokens = SpecialTokens(0, 1)) -> Generator[torch.Tensor, None, None]:
        with torch.inference_mode():
            with stats.text_generation(ledger) as r:
                for output_tokens in self._generate(r, input_ids, max_length, beam_shape, sampling_args, special_tokens):
                    yield output_tokens

    # ------------------------------------------------------------------------------------------
    def _comprehend_prompt(self, st: _DecodeState, cache: kv_cache.Cache, input_ids: torch.Tensor,
                           sampling_args: SamplingArgs, pad_token_id: int) -> int:
        """Prefill (recurrent_drafting.py:391-434) over the non-pad tokens only.  Fills the cache,
        st.ctx (hidden state of every row's last token) and st.init_tok.  Returns max row length."""
        llm = self.llm
        B, Lp = input_ids.shape
        dev = input_ids.device
        pads = _count_left_paddings(input_ids, pad_token_id)
        n_new = Lp - pads
        assert int(n_new.min().item()) >= 1, "a prompt row holds only padding"
        cols = torch.arange(Lp, device=dev)[None, :].expand(B, Lp)
        live = cols >= pads[:, None]
        tok_ids = input_ids[live].contiguous()
        M = tok_ids.numel()
        tok_row = torch.arange(B, device=dev)[:, None].expand(B, Lp)[live].to(torch.int32)
        tok_pos = (cols - pads[:, None])[live].to(torch.int32)
        tok_slot = tok_pos  # rows are stored without their left padding: slot = position
        row_start = torch.zeros(B + 1, dtype=torch.int32, device=dev)
        row_start[1:] = torch.cumsum(n_new, 0).to(torch.int32)
        st.kv_begin.zero_()
        base_len = torch.zeros(B, dtype=torch.int32, device=dev)
        ws = llm.workspace(M, B)
        hidden = llm.backbone(ws, cache._cache, M, None, tok_ids, tok_row, tok_pos, tok_slot, row_start, st.kv_begin,
                              base_len, B, Lp, Lp, _lib.ATTN_CAUSAL, n_pos=cache._cache.shape[4] + 1)
        last = (row_start[1:] - 1).long()
        st.ctx.copy_(hidden[last])
        logits = llm.lm_logits(st.ctx, ws["logits"])
        V = logits.shape[1]
        if sampling_args.greedy:
            _lib.call("rd_argmax_rows", _lib.ptr(logits), logits.stride(0), B, None, V, None, _lib.ptr(st.init_tok), _lib.stream())
        else:
            sp = modeling_drafter.vocab_topk(logits, modeling_drafter.new_sparse(B, dev), subtract_max=False,
                                             temperature=sampling_args.temperature)
            u = torch.rand(B, device=dev)
            _lib.call("rd_sample_from_sparse", _lib.ptr(sp.val), _lib.ptr(sp.idx), _lib.ptr(sp.cnt), B, _lib.ptr(u),
                      _lib.ptr(st.init_tok), _lib.stream())
        st.kv_len.copy_(n_new.to(torch.int32))
        # the same compaction for the token ids: column c of row b holds input_ids[b, pads[b] + c]
        st.token_buf[:, :Lp] = torch.gather(input_ids, 1, (cols + pads[:, None]).clamp_(max=Lp - 1))
        for k, v in cache.sliced:
            k.length = v.length = Lp
        return int(n_new.max().item())

    # One decode step = three phases that enqueue kernels and never synchronise with the host
    # (recurrent_drafting.py:626-679).  They take and return only tensors that live as long as the generate()
    # call, so each phase can also be captured once into a CUDA graph and replayed (see _StepGraphs).
    def _draft_phase(self, st: _DecodeState, beam_shape) -> modeling_drafter.DraftResult:
        return self.drafter.beam_search_sparse(st.ctx, st.init_tok, self.llm.get_input_embeddings(), beam_shape)

    def _verify_phase(self, st: _DecodeState, cache: kv_cache.Cache, beam_shape, sampling_args: SamplingArgs,
                      draft: modeling_drafter.DraftResult, s_max: int, rec=None):
        llm = self.llm
        B = st.kv_begin.shape[0]
        W, Lb = beam_shape.width, beam_shape.length
        cache_t = cache._cache
        max_len = cache_t.shape[4]
        fp = tree_attention.pack_flat(draft.beams, st.kv_begin, st.kv_len, out=st.fp)
        m_max = B * W * Lb
        ws = llm.workspace(m_max, m_max)
        with (rec.time("base_forward") if rec is not None else contextlib.nullcontext()):
            # On the tensor-core path the bound on the keys only decides the key-range split of the attention; it is
            # taken from the cache's capacity there, so that every step of a request launches the same kernels.
            # The CUDA-core attention sizes its shared memory by it and gets the tight bound.
            tc_path = llm.dtype == torch.bfloat16 and llm.head_dim == 128
            max_kv = max_len if tc_path else s_max + W * Lb
            hidden = llm.backbone(ws, cache_t, m_max, fp.m_dev, fp.tokens, fp.tok_row, fp.tok_pos, fp.tok_slot,
                                  fp.row_start, st.kv_begin, fp.base_len, B, W * Lb, max_kv, _lib.ATTN_TREE,
                                  tree_mask=fp.tree_mask, mask_words=fp.mask_words, n_pos=max_len + 1)
            fused_head = llm.fused_head_ok()
            smax = None
            if sampling_args.greedy and fused_head:
                # the arg-max over the vocabulary rides on the LM head's epilogue: no logits are written
                llm.lm_argmax(hidden, st.llm_tok, m_dev=fp.m_dev)
                logits = ws["logits"]
            elif sampling_args.greedy:
                logits = llm.lm_logits(hidden, ws["logits"], m_dev=fp.m_dev)
            else:
                logits = ws["logits"]
                smax = llm.lm_logits_with_slice_max(hidden, logits, m_dev=fp.m_dev)
        return fp, hidden, logits, smax, fused_head

    def _accept_phase(self, st: _DecodeState, cache: kv_cache.Cache, beam_shape, sampling_args: SamplingArgs,
                      draft: modeling_drafter.DraftResult, verified) -> None:
        llm = self.llm
        fp, hidden, logits, smax, fused_head = verified
        B = st.kv_begin.shape[0]
        W, Lb = beam_shape.width, beam_shape.length
        code = _lib.dtype_code(llm.dtype)
        sm = _lib.stream()
        cache_t = cache._cache
        NL, _, _, nkv, max_len, hd = cache_t.shape
        H = llm.config.hidden_size
        m_max = B * W * Lb
        V = logits.shape[1]
        if sampling_args.greedy:
            if not fused_head:
                _lib.call("rd_argmax_rows", _lib.ptr(logits), logits.stride(0), m_max, _lib.ptr(fp.m_dev), V,
                          _lib.ptr(st.llm_tok), None, sm)
            _lib.call("rd_accept_commit_greedy", code, _lib.ptr(draft.beams), B, W, Lb, _lib.ptr(fp.unpacker),
                      _lib.ptr(fp.row_start), _lib.ptr(st.llm_tok), _lib.ptr(hidden), H, _lib.ptr(cache_t), NL, nkv,
                      max_len, hd, _lib.ptr(st.kv_begin), _lib.ptr(fp.base_len), _lib.ptr(st.kv_len),
                      _lib.ptr(st.token_buf), _lib.ptr(st.n_accepted), _lib.ptr(st.seq_in_beam), _lib.ptr(st.init_tok),
                      _lib.ptr(st.ctx), sm)
        else:
            modeling_drafter.vocab_topk(logits, st.p, subtract_max=False, temperature=sampling_args.temperature,
                                        rows_dev=fp.m_dev, slice_max=smax)
            u, u_next = st.u, st.u_next  # drawn by _step before this phase
            q = draft.q
            _lib.call("rd_accept_commit_sample", code, _lib.ptr(draft.beams), B, W, Lb, V, _lib.ptr(fp.unpacker),
                      _lib.ptr(fp.row_start), _lib.ptr(st.p.val), _lib.ptr(st.p.idx), _lib.ptr(st.p.cnt),
                      _lib.ptr(st.p.masked), _lib.ptr_array([x.val for x in q]), _lib.ptr_array([x.idx for x in q]),
                      _lib.ptr_array([x.cnt for x in q]), _lib.ptr_array([x.masked for x in q]), _lib.ptr(draft.anc),
                      _lib.ptr(u), _lib.ptr(u_next), _lib.ptr(hidden), H, _lib.ptr(cache_t), NL, nkv, max_len, hd,
                      _lib.ptr(st.kv_begin), _lib.ptr(fp.base_len), _lib.ptr(st.kv_len), _lib.ptr(st.token_buf),
                      _lib.ptr(st.n_accepted), _lib.ptr(st.seq_in_beam), _lib.ptr(st.init_tok), _lib.ptr(st.ctx),
                      None, sm)

    def _step(self, st: _DecodeState, cache: kv_cache.Cache, beam_shape, sampling_args: SamplingArgs, s_max: int,
              rec: stats.TextGeneration.Step, graphs: Optional["_StepGraphs"] = None) -> None:
        """Enqueues one decode step.  No host synchronisation."""
        if not sampling_args.greedy:
            st.draw_uniforms(st.kv_begin.shape[0], beam_shape.width, beam_shape.length)
        if graphs is not None and graphs.ready:
            with rec.time("generate_candidates"):
                graphs.draft.replay()
            with rec.time("verify_candidates"):
                graphs.verify.replay()
            with rec.time("accept_candidate_tokens"):
                graphs.accept.replay()
            _lib.count_replay(graphs.n_kernels)
            return
        with rec.time("generate_candidates"):
            draft = self._draft_phase(st, beam_shape)
        with rec.time("verify_candidates"):
            verified = self._verify_phase(st, cache, beam_shape, sampling_args, draft, s_max, rec)
        with rec.time("accept_candidate_tokens"):
            self._accept_phase(st, cache, beam_shape, sampling_args, draft, verified)

    def _graphs_apply(self, sampling_args: SamplingArgs) -> bool:
        """CUDA graphs are used on the tensor-core path when enabled (the uniforms of a sampling step are drawn
        outside the graphs, from torch's generator as without them)."""
        llm = self.llm
        return bool(self.cuda_graphs and llm.dtype == torch.bfloat16 and llm.head_dim == 128 and llm.fused_head_ok())

    def _generate(self, text_generation: stats.TextGeneration, input_ids: torch.Tensor, max_length: int,
                  beam_shape: modeling_drafter.BeamShape, sampling_args: SamplingArgs,
                  special_tokens: SpecialTokens) -> Generator[torch.Tensor, None, None]:
        assert input_ids.dtype == torch.long, f"input_ids.dtype {input_ids.dtype} is not long"
        if not input_ids.is_cuda:
            raise _lib.RedrafterError("input_ids must live on a CUDA device: this package has no CPU path")
        llm = self.llm
        B, seq_len = input_ids.shape
        init_seq_len = seq_len
        W, Lb = beam_shape.width, beam_shape.length
        dev = input_ids.device
        cache = kv_cache.Cache(
            batch_size=B,
            max_length=max_length + Lb * W,
            n_layers=llm.n_layers,
            n_heads=self.llm_n_kv_heads(),
            head_dim=llm.head_dim,
            dtype=llm.dtype,
            device=dev,
        )
        st = _DecodeState(llm, B, W, Lb, max_length + Lb * W, dev)
        llm.gemm_status = st.status
        self.last_state = st
        self.last_cache = cache
        assert max_length + Lb * W <= st.token_buf.shape[1] == cache._cache.shape[4]
        s_max = self._comprehend_prompt(st, cache, input_ids, sampling_args, special_tokens.pad)
        ref_len = seq_len  # the reference's padded sequence length S before the step
        graphs = _StepGraphs() if self._graphs_apply(sampling_args) else None
        n_steps = 0
        while seq_len < max_length:
            if graphs is not None and not graphs.ready and n_steps == 2:
                # replayed from this step on (the first two ran eagerly: every descriptor set and workspace exists)
                graphs.capture(self, st, cache, beam_shape, sampling_args)
            n_steps += 1
            with text_generation.step() as rec:
                self._step(st, cache, beam_shape, sampling_args, s_max, rec, graphs)
                st.small_host.copy_(st.small, non_blocking=True)
                torch.cuda.current_stream().synchronize()
                if int(st.small_host[2, 0]) != 0:
                    raise _lib.RedrafterError(
                        f"a tensor-core kernel gave up waiting on its pipeline (status {int(st.small_host[2, 0])})")
                s_max = int(st.small_host[0].max())
                # rows are left-compacted, so the next step writes at most W*Lb slots past the longest row
                assert s_max + W * Lb <= st.token_buf.shape[1] or s_max + 1 >= max_length
                out = torch.empty(B, s_max + 1, dtype=torch.int64, device=dev)
                _lib.call("rd_emit_tokens", _lib.ptr(st.token_buf), st.token_buf.shape[1], _lib.ptr(st.kv_begin),
                          _lib.ptr(st.kv_len), _lib.ptr(st.init_tok), int(special_tokens.pad), B, s_max + 1, _lib.ptr(out),
                          _lib.stream())
                self.last_ref_lengths = (ref_len, s_max)
                ref_len = s_max
                for k, v in cache.sliced:
                    k.length = v.length = s_max
                seq_len = out.shape[1]
                rec.set({"input_id_length": seq_len, "avg_num_accepted": int(st.small_host[1].sum()) / B})
                yield out[:, :max_length] if seq_len > max_length else out
                if special_tokens.eos is not None and bool(
                    ((out[:, init_seq_len:] == special_tokens.eos).sum(dim=-1) > 0).sum() == B
                ):
                    break
        if int(st.status.item()) != 0:
            raise _lib.RedrafterError(f"a tensor-core GEMM gave up waiting on its pipeline (status {int(st.status.item())})")

    def reference_commit_slots(self, beam_shape: modeling_drafter.BeamShape) -> torch.Tensor:
        """[B, Lb, 3] int64: the last step's commit in the reference's right-aligned slot numbering
        (source slot after the verify forward, after Cache.unpack, and final slot)."""
        st = self.last_state
        B = st.kv_begin.shape[0]
        W, Lb = beam_shape.width, beam_shape.length
        S, S2 = self.last_ref_lengths
        out = torch.empty(B, Lb, 3, dtype=torch.int64, device=st.kv_begin.device)
        _lib.call("rd_commit_reference_slots", B, W, Lb, _lib.ptr(st.fp.unpacker), _lib.ptr(st.n_accepted),
                  _lib.ptr(st.seq_in_beam), S, S2, _lib.ptr(out), _lib.stream())
        return out
