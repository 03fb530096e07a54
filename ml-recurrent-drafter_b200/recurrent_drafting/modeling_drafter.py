"""Recurrent drafter head and its beam search on the B200 kernels, with the reference's interface
(recurrent_drafting/modeling_drafter.py): Drafter(cfg).beam_search_candidates(prompt_state,
init_token, embeddings, beam_shape) -> (beams, log_probs); parameter names input_proj,
lm_head.{r}.linear, lm_head.{R}, rnn_u, rnn_w.

One beam-search iteration is: stage [embed(token) | parent state] -> one GEMM against the
concatenated [rnn_w | rnn_u] weight with bias + SiLU epilogue (the recurrent update) -> residual
blocks as GEMMs with bias + SiLU + residual epilogue -> vocabulary GEMM -> per-row top-50 warp +
log-softmax with sparse output -> cross-beam top-W and beam reorder.  The (batch, beam, Lb-1, vocab)
log-prob tensor of the reference is never materialised on the decode path; it is rebuilt from the
sparse lists only when a caller asks for it.
"""
import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import transformers

from . import _lib, configuration_drafter
from .modeling_llama import _Linear

LOG_0 = -50000.0
LOG_1 = 0.0
TOP_K = 50


@dataclass
class BeamShape:
    width: int
    length: int


def register_auto_models() -> None:
    transformers.AutoConfig.register(
        model_type=configuration_drafter.DrafterConfig.model_type, config=configuration_drafter.DrafterConfig
    )
    transformers.AutoModel.register(config_class=configuration_drafter.DrafterConfig, model_class=Drafter)


class ResBlock(torch.nn.Module):
    """x + silu(linear(x)); evaluated inside a GEMM epilogue on the decode path (modeling_drafter.py:33-39)."""

    def __init__(self, cfg):
        super().__init__()
        self.linear = torch.nn.Linear(cfg.exit_dim, cfg.exit_dim, bias=True)


@dataclass
class SparseLogProbs:
    """Sparse form of log-softmax(warp_logits(.)) rows: per row the kept (>= top-50) entries'
    log-probs and vocabulary ids, their count, and the log-prob shared by all other entries."""

    val: torch.Tensor  # [rows, 64] fp32
    idx: torch.Tensor  # [rows, 64] int32
    cnt: torch.Tensor  # [rows] int32
    masked: torch.Tensor  # [rows] fp32


def vocab_topk(logits: torch.Tensor, out: SparseLogProbs, subtract_max: bool, temperature: float = 1.0,
               rows_dev: Optional[torch.Tensor] = None, top_k: int = TOP_K, mask_value: float = LOG_0,
               slice_max: Optional[torch.Tensor] = None) -> SparseLogProbs:
    """Sparse log-softmax(warp(logits)) rows.  slice_max [V/32, >= rows], when the GEMM that produced the
    logits also wrote it, lets the kernel read only the slices that can hold kept entries."""
    rows, V = logits.shape
    if slice_max is not None:
        _lib.call("rd_vocab_topk_sliced", _lib.dtype_code(logits.dtype), _lib.ptr(logits), logits.stride(0), rows, _lib.ptr(rows_dev),
                  V, min(top_k, V), mask_value, int(subtract_max), float(temperature), _lib.ptr(slice_max), slice_max.stride(0),
                  _lib.ptr(out.val), _lib.ptr(out.idx), _lib.ptr(out.cnt), _lib.ptr(out.masked), _lib.stream())
        return out
    _lib.call("rd_vocab_topk", _lib.dtype_code(logits.dtype), _lib.ptr(logits), logits.stride(0), rows, _lib.ptr(rows_dev), V,
              min(top_k, V), mask_value, int(subtract_max), float(temperature), _lib.ptr(out.val), _lib.ptr(out.idx),
              _lib.ptr(out.cnt), _lib.ptr(out.masked), _lib.stream())
    return out


def new_sparse(rows: int, device) -> SparseLogProbs:
    K = _lib.TOPK_MAX_KEPT
    return SparseLogProbs(
        torch.empty(rows, K, dtype=torch.float32, device=device),
        torch.empty(rows, K, dtype=torch.int32, device=device),
        torch.empty(rows, dtype=torch.int32, device=device),
        torch.empty(rows, dtype=torch.float32, device=device),
    )


def _dense_from_sparse(sp: SparseLogProbs, V: int) -> torch.Tensor:
    rows = sp.cnt.shape[0]
    anc = torch.arange(rows, dtype=torch.int32, device=sp.val.device).reshape(1, rows, 1)
    out = torch.empty(1, rows, 1, V, dtype=torch.float32, device=sp.val.device)
    _lib.call("rd_drafter_dense_log_probs", 1, rows, 2, V, _lib.ptr_array([sp.val]), _lib.ptr_array([sp.idx]),
              _lib.ptr_array([sp.cnt]), _lib.ptr_array([sp.masked]), _lib.ptr(anc), _lib.ptr(out), _lib.stream())
    return out.reshape(rows, V)


def maintain_logits(logits: torch.Tensor) -> torch.Tensor:
    """logits - row max (modeling_drafter.py:63-77).  Dense API helper; the decode path fuses this
    into rd_vocab_topk."""
    return logits - logits.max(dim=-1, keepdim=True)[0]


def warp_logits(logits: torch.Tensor, top_k: int = TOP_K, mask_value: float = LOG_0) -> torch.Tensor:
    """Keeps every value >= the top_k-th largest of its row, sets the rest to mask_value
    (modeling_drafter.py:80-99).  Computed by rd_vocab_topk (threshold) on the device."""
    shape = logits.shape
    flat = logits.reshape(-1, shape[-1]).contiguous()
    sp = vocab_topk(flat if flat.dtype in (torch.float32, torch.bfloat16) else flat.float(),
                    new_sparse(flat.shape[0], logits.device), subtract_max=False, top_k=top_k, mask_value=mask_value)
    # kept ids -> boolean keep mask; the values themselves are untouched
    keep = torch.zeros(flat.shape, dtype=torch.bool, device=logits.device)
    valid = torch.arange(_lib.TOPK_MAX_KEPT, device=logits.device)[None, :] < sp.cnt[:, None]
    rows = torch.arange(flat.shape[0], device=logits.device)[:, None].expand_as(sp.idx)
    keep[rows[valid], sp.idx[valid].long()] = True
    return torch.where(keep, flat, torch.full_like(flat, mask_value)).reshape(shape)


@dataclass
class DraftResult:
    beams: torch.Tensor  # [B, W, Lb] int64
    q: List[SparseLogProbs]  # Lb-1 lists over rows b*W + beam-at-that-iteration
    anc: torch.Tensor  # [B, W, Lb-1] int32 ancestor row (within the batch row) per iteration


class Drafter(torch.nn.Module):
    config_class = configuration_drafter.DrafterConfig

    def __init__(self, cfg: configuration_drafter.DrafterConfig):
        super().__init__()
        self.config = cfg
        input_dim = 2 * cfg.hidden_size
        if input_dim != cfg.exit_dim:
            self.input_proj = torch.nn.Linear(input_dim, cfg.exit_dim, bias=True)
        self.lm_head = torch.nn.Sequential(
            *[ResBlock(cfg) for _ in range(cfg.num_draft_layers)],
            torch.nn.Linear(cfg.exit_dim, cfg.vocab_size, bias=False),
        )
        if cfg.rnn:
            self.rnn_u = torch.nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=True)
            self.rnn_w = torch.nn.Linear(cfg.hidden_size, cfg.hidden_size, bias=False)
        for prm in self.parameters():
            prm.requires_grad_(False)
        self._packed = None
        self._ws: Dict[Tuple, Dict] = {}

    @property
    def dtype(self) -> torch.dtype:
        return self.lm_head[-1].weight.dtype

    @property
    def device(self) -> torch.device:
        return self.lm_head[-1].weight.device

    def init_random(self, std: float = 0.02, seed: int = 1) -> "Drafter":
        g = torch.Generator(device=self.device).manual_seed(seed)
        for prm in self.parameters():
            prm.copy_(torch.randn(prm.shape, generator=g, device=prm.device, dtype=torch.float32).mul_(std))
        self._invalidate()
        return self

    @classmethod
    def from_pretrained(cls, path: str, torch_dtype: torch.dtype = torch.bfloat16, device="cuda") -> "Drafter":
        """A drafter checkpoint directory as written by the reference's training code (config.json of
        model_type recurrent_drafting_drafter + weights under the reference's parameter names)."""
        from . import checkpoint

        cfg = configuration_drafter.DrafterConfig.from_pretrained(path)
        model = cls(cfg)
        ck = checkpoint.LazyCheckpoint(path)
        model.load_state_dict({k: ck.pop(k) for k in ck.keys()})
        return model.to(device=device, dtype=torch_dtype)

    def save_pretrained(self, path: str) -> None:
        from . import checkpoint

        checkpoint.save_directory(path, self.config, self.state_dict())

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        out = super().load_state_dict(state_dict, strict=strict)
        self._invalidate()
        return out

    def _apply(self, fn, *args, **kwargs):
        out = super()._apply(fn, *args, **kwargs)
        self._invalidate()
        return out

    def _invalidate(self):
        self._packed = None
        self._ws = {}

    def _lin(self):
        if self._packed is None:
            R = self.config.num_draft_layers
            self._packed = {
                # [emb | state] @ [rnn_w | rnn_u]^T + b_u  == rnn_w(emb) + rnn_u(state); a drafter built with
                # rnn=False has no such projections (its state update is embedding + state)
                "rnn": _Linear(torch.cat([self.rnn_w.weight, self.rnn_u.weight], dim=1).contiguous(), self.rnn_u.bias)
                if self.config.rnn else None,
                "res": [_Linear(self.lm_head[r].linear.weight, self.lm_head[r].linear.bias) for r in range(R)],
                "vocab": _Linear(self.lm_head[R].weight),
                "proj": _Linear(self.input_proj.weight, self.input_proj.bias) if hasattr(self, "input_proj") else None,
            }
        return self._packed

    def _workspace(self, B: int, W: int, Lb: int) -> Dict:
        key = (B, W, Lb)
        ws = self._ws.get(key)
        if ws is None:
            cfg, dt, dev = self.config, self.dtype, self.device
            H, E, V = cfg.hidden_size, cfg.exit_dim, cfg.vocab_size
            M = B * W
            e = lambda *s, d=dt: torch.empty(*s, dtype=d, device=dev)  # noqa: E731
            ws = {
                "a": e(M, 2 * H),
                "x": e(M, 2 * H),
                "y": [e(M, E), e(M, E), e(M, E)],
                "logits": e(M, V),
                # per-(32 vocabulary ids, row) maxima written by the vocabulary GEMM's epilogue
                "slice_max": e(V // 32, (M + 31) // 32 * 32, d=torch.float32) if V % 32 == 0 else None,
                "q": [new_sparse(M, dev) for _ in range(Lb - 1)],
                "q_first": new_sparse(B, dev),  # the first iteration's lists, one per batch row
                "score": [e(B, W, d=torch.float32), e(B, W, d=torch.float32)],
                "beams": [torch.zeros(B, W, Lb, dtype=torch.int64, device=dev) for _ in range(2)],
                "anc": [torch.zeros(B, W, max(Lb - 1, 1), dtype=torch.int32, device=dev) for _ in range(2)],
                "parent": torch.zeros(B, W, dtype=torch.int32, device=dev),
            }
            if len(self._ws) >= 4:  # a few (batch, beam shape) combinations at most stay resident
                self._ws.pop(next(iter(self._ws)))
                for lin in self._lin().values():
                    for one in (lin if isinstance(lin, list) else [lin]):
                        if one is not None:
                            one.drop_plans()
            self._ws[key] = ws
        return ws

    def compute_logits(self, x: torch.Tensor) -> torch.Tensor:
        """Dense warped logits of LM-head inputs x (..., 2H) (modeling_drafter.py:127-131)."""
        lin = self._lin()
        shape = x.shape
        cur = x.reshape(-1, shape[-1]).contiguous()
        M = cur.shape[0]
        E, V = self.config.exit_dim, self.config.vocab_size
        if lin["proj"] is not None:
            nxt = torch.empty(M, E, dtype=cur.dtype, device=cur.device)
            lin["proj"](cur, nxt, _lib.EPI_BIAS)
            cur = nxt
        for res in lin["res"]:
            nxt = torch.empty(M, E, dtype=cur.dtype, device=cur.device)
            res(cur, nxt, _lib.EPI_BIAS_SILU_RES, residual=cur)
            cur = nxt
        logits = torch.empty(M, V, dtype=cur.dtype, device=cur.device)
        lin["vocab"](cur, logits)
        return warp_logits(maintain_logits(logits)).reshape(*shape[:-1], V)

    @torch.inference_mode()
    def beam_search_sparse(self, prompt_state: torch.Tensor, init_token: torch.Tensor, embeddings: torch.nn.Embedding,
                           beam_shape: BeamShape) -> DraftResult:
        """The decode-path beam search: kernels only, no host synchronisation."""
        assert init_token.dtype == torch.long and prompt_state.ndim == 2 and init_token.ndim == 1
        assert beam_shape.length > 1
        B, H = prompt_state.shape
        W, Lb = beam_shape.width, beam_shape.length
        assert W <= _lib.MAX_BEAM_WIDTH and Lb <= _lib.MAX_BEAM_LENGTH
        cfg = self.config
        V = cfg.vocab_size
        assert embeddings.weight.shape == (V, H) and embeddings.weight.dtype == self.dtype
        lin = self._lin()
        ws = self._workspace(B, W, Lb)
        code = _lib.dtype_code(self.dtype)
        st = _lib.stream()
        a, x = ws["a"], ws["x"]
        ws["beams"][0][:, :, 0] = init_token[:, None]
        ctx = prompt_state.contiguous()
        for k in range(Lb - 1):
            bin_, bout = ws["beams"][k % 2], ws["beams"][(k + 1) % 2]
            _lib.call("rd_drafter_prepare", code, _lib.ptr(embeddings.weight), _lib.ptr(bin_), _lib.ptr(ws["parent"]),
                      _lib.ptr(ctx), _lib.ptr(a), _lib.ptr(x), B, W, Lb, H, k, 0 if cfg.rnn else 1, st)
            # In the first iteration every beam of a row holds the same token, state and context
            # (modeling_drafter.py:170-177), so the W rows of a batch row are identical: compute row 0
            # of each (a view with row stride W) and copy its results to the others.
            shared = k == 0 and W > 1
            rows = slice(None, None, W) if shared else slice(None)
            a_k, x_k, ys, logits_k = a[rows], x[rows], [y[rows] for y in ws["y"]], ws["logits"][rows]
            q_k = ws["q_first"] if shared else ws["q"][k]
            # recurrent update, written into the state half of x
            if lin["rnn"] is not None:
                lin["rnn"](a_k, x_k[:, H:], _lib.EPI_BIAS_SILU, ldc=x_k.stride(0))
            else:
                x_k[:, H:].copy_(a_k[:, H:])  # the prepare kernel already formed embedding + parent state
            cur = x_k
            yi = 0
            if lin["proj"] is not None:
                lin["proj"](cur, ys[yi], _lib.EPI_BIAS)
                cur, yi = ys[yi], yi + 1
            for res in lin["res"]:
                nxt = ys[yi % 3]
                res(cur, nxt, _lib.EPI_BIAS_SILU_RES, residual=cur)
                cur, yi = nxt, yi + 1
            smax = ws["slice_max"] if os.environ.get("RD_FUSED_HEAD", "1") != "0" else None
            if smax is not None and not shared and lin["vocab"].with_slice_max(cur, logits_k, smax):
                vocab_topk(logits_k, q_k, subtract_max=True, slice_max=smax)
            else:
                lin["vocab"](cur, logits_k)
                vocab_topk(logits_k, q_k, subtract_max=True)
            if shared:
                q = ws["q"][0]
                K = q.val.shape[1]
                q.val.view(B, W, K).copy_(q_k.val.view(B, 1, K).expand(B, W, K))
                q.idx.view(B, W, K).copy_(q_k.idx.view(B, 1, K).expand(B, W, K))
                q.cnt.view(B, W).copy_(q_k.cnt.view(B, 1).expand(B, W))
                q.masked.view(B, W).copy_(q_k.masked.view(B, 1).expand(B, W))
                xs = x.view(B, W, 2 * H)
                xs[:, 1:, H:].copy_(xs[:, :1, H:].expand(B, W - 1, H))
            _lib.call("rd_beam_select", B, W, Lb, k, V, _lib.ptr(ws["q"][k].val), _lib.ptr(ws["q"][k].idx),
                      _lib.ptr(ws["q"][k].cnt), _lib.ptr(ws["score"][k % 2]), _lib.ptr(ws["score"][(k + 1) % 2]),
                      _lib.ptr(bin_), _lib.ptr(bout), _lib.ptr(ws["anc"][k % 2]), _lib.ptr(ws["anc"][(k + 1) % 2]),
                      _lib.ptr(ws["parent"]), st)
        last = (Lb - 1) % 2
        return DraftResult(ws["beams"][last], ws["q"], ws["anc"][last])

    @torch.inference_mode()
    def beam_search_candidates(self, prompt_state: torch.Tensor, init_token: torch.Tensor, embeddings: torch.nn.Embedding,
                               beam_shape: BeamShape = BeamShape(10, 4)) -> Tuple[torch.Tensor, torch.Tensor]:
        """Reference signature (modeling_drafter.py:133-232): returns beams (B,W,Lb) int64 and the
        dense log-probs (B,W,Lb-1,V) fp32."""
        r = self.beam_search_sparse(prompt_state, init_token, embeddings, beam_shape)
        B, W, Lb = r.beams.shape
        V = self.config.vocab_size
        out = torch.empty(B, W, Lb - 1, V, dtype=torch.float32, device=r.beams.device)
        _lib.call("rd_drafter_dense_log_probs", B, W, Lb, V, _lib.ptr_array([q.val for q in r.q]),
                  _lib.ptr_array([q.idx for q in r.q]), _lib.ptr_array([q.cnt for q in r.q]),
                  _lib.ptr_array([q.masked for q in r.q]), _lib.ptr(r.anc), _lib.ptr(out), _lib.stream())
        return r.beams.clone(), out
