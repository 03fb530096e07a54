"""Llama-architecture base model on the B200 kernels, with the reference's interface
(recurrent_drafting/modeling_llama.py): LlamaForCausalLM(config).forward(input_ids, attention_mask,
position_ids, past_key_values) -> CausalLMOutput(logits fp32, hidden_states), HF state-dict names.

Weights are held in the layouts the kernels consume: q/k/v projections concatenated into one
[(nh+2*nkv)*hd, H] matrix, gate/up projections row-interleaved into one [2*I, H] matrix so that the
SwiGLU product is formed in the GEMM epilogue.  load_state_dict()/state_dict() translate from and
to the HF names (model.layers.N.self_attn.q_proj.weight, ...).

Two entry points share one token-major implementation:
  * forward(): the reference's padded (batch, q_len) call with an explicit bool mask;
  * forward_tokens(): ragged rows packed back to back with per-row cache offsets and either causal
    or prefix-tree visibility; this is what the decode loop uses.
"""
import math
import os
from typing import Dict, Optional, Tuple

import torch
from torch import nn
from transformers.modeling_outputs import CausalLMOutput

from . import _lib, attention, checkpoint, kv_cache


class _Linear:
    """y = epilogue(x W^T) on a fixed weight; picks the tcgen05 path for bf16 when shapes allow."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.weight = weight
        self.bias = bias
        self._plans: Dict[Tuple, int] = {}

    MAX_PLANS = 32  # distinct (activation buffer, row capacity) pairs remembered per weight

    def drop_plans(self) -> None:
        plans, self._plans = self._plans, {}
        if plans:
            lib = _lib.load()
            for p in plans.values():
                lib.rd_gemm_plan_destroy(p)

    def __del__(self):
        try:
            self.drop_plans()
        except Exception:
            pass

    def _tc_ok(self, a: torch.Tensor, lda: int) -> bool:
        n, k = self.weight.shape
        return (
            self.weight.dtype == torch.bfloat16
            and k % 64 == 0
            and a.data_ptr() % 16 == 0
            and (lda * 2) % 16 == 0
            and self.weight.data_ptr() % 16 == 0
        )

    def _plan(self, a: torch.Tensor, lda: int, m_max: int) -> int:
        n, k = self.weight.shape
        key = (a.data_ptr(), lda, m_max)
        plan = self._plans.get(key)
        if plan is None:
            plan = _lib.load().rd_gemm_plan_create(_lib.ptr(a), lda, m_max, _lib.ptr(self.weight), self.weight.stride(0), n, k)
            if not plan:
                raise _lib.RedrafterError("rd_gemm_plan_create failed (TMA descriptor could not be encoded)")
            if len(self._plans) >= self.MAX_PLANS:
                self.drop_plans()
            self._plans[key] = plan
        return plan

    def qkv_rope(self, a: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, tok_row, tok_pos,
                 tok_slot, cos: torch.Tensor, sin: torch.Tensor, nh: int, nkv: int, hd: int, m_dev, m_max: int,
                 status: Optional[torch.Tensor], norm=None) -> None:
        """This weight as the packed QKV projection with rotary embedding and cache append in the
        GEMM epilogue (rd_gemm_bf16_tc_qkv_rope); tensor-core path only."""
        if not self._tc_ok(a, a.stride(0)):
            raise _lib.RedrafterError("the fused QKV projection needs the tensor-core GEMM path (bf16, aligned operands)")
        plan = self._plan(a, a.stride(0), m_max)
        if norm is not None:
            # `a` holds gamma-scaled, not normalised rows: the 1 / rms of each row is applied in the epilogue
            ss, dim, eps = norm
            _lib.call("rd_gemm_bf16_tc_qkv_rope_normed", plan, _lib.ptr(m_dev), _lib.ptr(q_out), _lib.ptr(k_cache),
                      _lib.ptr(v_cache), _lib.ptr(tok_row), _lib.ptr(tok_pos), _lib.ptr(tok_slot), _lib.ptr(cos), _lib.ptr(sin),
                      cos.shape[0], nh, nkv, hd, k_cache.shape[2], _lib.ptr(ss), ss.stride(0), dim // 128, dim, eps,
                      _lib.ptr(status), _lib.stream())
            return
        _lib.call("rd_gemm_bf16_tc_qkv_rope", plan, _lib.ptr(m_dev), _lib.ptr(q_out), _lib.ptr(k_cache), _lib.ptr(v_cache),
                  _lib.ptr(tok_row), _lib.ptr(tok_pos), _lib.ptr(tok_slot), _lib.ptr(cos), _lib.ptr(sin), cos.shape[0], nh, nkv,
                  hd, k_cache.shape[2], _lib.ptr(status), _lib.stream())

    def residual_with_norm(self, a: torch.Tensor, c: torch.Tensor, residual: torch.Tensor, gamma: torch.Tensor,
                           c2: torch.Tensor, ss: torch.Tensor, m_dev, m_max: int, status: Optional[torch.Tensor]) -> None:
        """c = a @ weight^T + residual, and the producer half of the RMS norm that follows: c2 = c * gamma and the
        per-slice sums of squares ss [m_max, >= features / 128] (rd_gemm_bf16_tc_res_norm); tensor-core path only."""
        if not self._tc_ok(a, a.stride(0)):
            raise _lib.RedrafterError("the folded RMS norm needs the tensor-core GEMM path (bf16, aligned operands)")
        plan = self._plan(a, a.stride(0), m_max)
        _lib.call("rd_gemm_bf16_tc_res_norm", plan, _lib.ptr(c), c.stride(0), _lib.ptr(residual), residual.stride(0),
                  _lib.ptr(m_dev), _lib.ptr(gamma), _lib.ptr(c2), c2.stride(0), _lib.ptr(ss), ss.stride(0), _lib.ptr(status),
                  _lib.stream())

    def swiglu_normed(self, a: torch.Tensor, c: torch.Tensor, ss: torch.Tensor, dim: int, eps: float, m_dev, m_max: int,
                      status: Optional[torch.Tensor]) -> None:
        """SwiGLU projection of rows that are gamma-scaled but not normalised: each row's 1 / rms, from the sums of
        squares ss, is applied in the epilogue (rd_gemm_bf16_tc_swiglu_normed); tensor-core path only."""
        if not self._tc_ok(a, a.stride(0)):
            raise _lib.RedrafterError("the folded RMS norm needs the tensor-core GEMM path (bf16, aligned operands)")
        plan = self._plan(a, a.stride(0), m_max)
        _lib.call("rd_gemm_bf16_tc_swiglu_normed", plan, _lib.ptr(c), c.stride(0), _lib.ptr(m_dev), _lib.ptr(ss), ss.stride(0),
                  dim // 128, dim, eps, _lib.ptr(status), _lib.stream())

    def argmax(self, a: torch.Tensor, out32: torch.Tensor, workspace: torch.Tensor, m_dev, m_max: int,
               status: Optional[torch.Tensor]) -> None:
        """out32[t] = argmax_n (a[t] . weight[n]) without materialising the product: the arg-max rides on
        the GEMM's epilogue (rd_gemm_bf16_tc_argmax); tensor-core path only."""
        if not self._tc_ok(a, a.stride(0)):
            raise _lib.RedrafterError("the fused LM-head arg-max needs the tensor-core GEMM path (bf16, aligned operands)")
        plan = self._plan(a, a.stride(0), m_max)
        _lib.call("rd_gemm_bf16_tc_argmax", plan, _lib.ptr(m_dev), _lib.ptr(workspace), workspace.numel(), _lib.ptr(out32), None,
                  _lib.ptr(status), _lib.stream())

    def with_slice_max(self, a: torch.Tensor, c: torch.Tensor, slice_max: torch.Tensor, m_dev=None, m_max: Optional[int] = None,
                       status: Optional[torch.Tensor] = None) -> bool:
        """c = a W^T plus the per-(32 outputs, row) maxima of c in slice_max [N/32, >= m_max]
        (rd_gemm_bf16_tc_slicemax).  Returns False, doing nothing, when the shapes rule it out."""
        n, k = self.weight.shape
        m_max = a.shape[0] if m_max is None else m_max
        esz = 4 if c.dtype == torch.float32 else 2
        if not (self._tc_ok(a, a.stride(0)) and n % 32 == 0 and c.data_ptr() % 16 == 0 and (c.stride(0) * esz) % 16 == 0
                and slice_max.shape[0] * 32 == n and slice_max.stride(0) >= m_max):
            return False
        plan = self._plan(a, a.stride(0), m_max)
        _lib.call("rd_gemm_bf16_tc_slicemax", plan, _lib.dtype_code(c.dtype), _lib.ptr(c), c.stride(0), _lib.ptr(m_dev),
                  _lib.ptr(slice_max), slice_max.stride(0), _lib.ptr(status), _lib.stream())
        return True

    def __call__(self, a: torch.Tensor, c: torch.Tensor, epilogue: int = _lib.EPI_NONE, residual=None,
                 m_dev: Optional[torch.Tensor] = None, lda: Optional[int] = None, ldc: Optional[int] = None,
                 ldr: Optional[int] = None, m_max: Optional[int] = None, status: Optional[torch.Tensor] = None) -> None:
        n, k = self.weight.shape
        m_max = a.shape[0] if m_max is None else m_max
        lda = a.stride(0) if lda is None else lda
        ldc = c.stride(0) if ldc is None else ldc
        if residual is not None and ldr is None:
            ldr = residual.stride(0)
        out_code = _lib.dtype_code(c.dtype)
        esz = 4 if c.dtype == torch.float32 else 2
        aligned = c.data_ptr() % 16 == 0 and (ldc * esz) % 16 == 0 and (
            residual is None or (residual.data_ptr() % 16 == 0 and (ldr * esz) % 16 == 0)
        )
        if self._tc_ok(a, lda) and aligned:
            plan = self._plan(a, lda, m_max)
            _lib.call("rd_gemm_bf16_tc", plan, out_code, _lib.ptr(c), ldc, _lib.ptr(self.bias), _lib.ptr(residual),
                      ldr or 0, _lib.ptr(m_dev), epilogue, _lib.ptr(status), _lib.stream())
        else:
            _lib.call("rd_gemm", _lib.dtype_code(self.weight.dtype), out_code, _lib.ptr(a), lda, _lib.ptr(self.weight),
                      self.weight.stride(0), _lib.ptr(c), ldc, _lib.ptr(self.bias), _lib.ptr(residual), ldr or 0, m_max,
                      _lib.ptr(m_dev), n, k, epilogue, _lib.stream())


def rope_tables(head_dim: int, n_pos: int, base: float, device) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 cos/sin tables [n_pos, head_dim], computed like LlamaRotaryEmbedding
    (modeling_llama.py:35-64) on the host and copied to the device."""
    inv_freq = 1.0 / (base ** (torch.arange(0, head_dim, 2).float() / head_dim))
    t = torch.arange(n_pos, dtype=inv_freq.dtype)
    freqs = torch.einsum("i,j->ij", t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().contiguous().to(device), emb.sin().contiguous().to(device)


class _Embedding(nn.Embedding):
    pass


class LlamaModel(nn.Module):
    """Holds embed_tokens so that `llm.base_model.get_input_embeddings()` works as in the reference."""

    def __init__(self, config):
        super().__init__()
        self.embed_tokens = _Embedding(config.vocab_size, config.hidden_size)

    def get_input_embeddings(self):
        return self.embed_tokens


class LlamaForCausalLM(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        H = config.hidden_size
        self.n_heads = config.num_attention_heads
        self.n_kv_heads = getattr(config, "num_key_value_heads", None) or self.n_heads
        self.head_dim = H // self.n_heads
        assert self.head_dim * self.n_heads == H
        self.n_layers = config.num_hidden_layers
        inter = config.intermediate_size
        self.rope_theta = float(getattr(config, "rope_theta", None) or 10000.0)
        self.eps = float(config.rms_norm_eps)
        qkv_rows = (self.n_heads + 2 * self.n_kv_heads) * self.head_dim
        self.model = LlamaModel(config)

        def p(*shape):
            return nn.Parameter(torch.empty(*shape), requires_grad=False)

        self.wqkv = nn.ParameterList([p(qkv_rows, H) for _ in range(self.n_layers)])
        self.wo = nn.ParameterList([p(H, self.n_heads * self.head_dim) for _ in range(self.n_layers)])
        self.wgu = nn.ParameterList([p(2 * inter, H) for _ in range(self.n_layers)])
        self.wdown = nn.ParameterList([p(H, inter) for _ in range(self.n_layers)])
        self.ln1 = nn.ParameterList([p(H) for _ in range(self.n_layers)])
        self.ln2 = nn.ParameterList([p(H) for _ in range(self.n_layers)])
        self.norm = p(H)
        self.lm_head = nn.Linear(H, config.vocab_size, bias=False)
        self.lm_head.weight.requires_grad_(False)
        self.model.embed_tokens.weight.requires_grad_(False)
        self._ws: Dict[Tuple, Dict[str, torch.Tensor]] = {}
        self._ws_full: Optional[Dict[str, torch.Tensor]] = None
        self._ws_cap: Tuple[int, int] = (0, 0)
        self._linears = None
        self._rope = None
        self._attn_plans: Dict[Tuple, int] = {}
        self._attn_split_ws: Optional[torch.Tensor] = None
        self._head_ws: Optional[torch.Tensor] = None
        self.gemm_status: Optional[torch.Tensor] = None

    # ----------------------------------------------------------------- reference-compatible surface
    @property
    def base_model(self):
        return self.model

    @property
    def dtype(self) -> torch.dtype:
        return self.lm_head.weight.dtype

    @property
    def device(self) -> torch.device:
        return self.lm_head.weight.device

    def get_input_embeddings(self):
        return self.model.embed_tokens

    def get_output_embeddings(self):
        return self.lm_head

    def init_random(self, std: float = 0.02, seed: int = 0) -> "LlamaForCausalLM":
        """Random-init weights in place (normal(0, std); norm weights 1), on the current device."""
        g = torch.Generator(device=self.device).manual_seed(seed)
        for prm in self.parameters():
            if prm.ndim == 1:
                prm.fill_(1.0)
            else:
                prm.copy_(torch.randn(prm.shape, generator=g, device=prm.device, dtype=torch.float32).mul_(std))
        self._invalidate()
        return self

    def load_state_dict(self, state_dict, strict: bool = True, assign: bool = False):
        """Accepts the HF / reference names and packs them into the kernel layouts."""
        sd = state_dict if isinstance(state_dict, checkpoint.LazyCheckpoint) else dict(state_dict)
        if any(k.startswith("wqkv.") for k in sd):
            out = super().load_state_dict(sd, strict=strict)
            self._invalidate()
            return out

        def take(name):
            return sd.pop(name).to(device=self.device, dtype=self.dtype)

        with torch.no_grad():
            self.model.embed_tokens.weight.copy_(take("model.embed_tokens.weight"))
            for l in range(self.n_layers):
                pre = f"model.layers.{l}."
                self.wqkv[l].copy_(torch.cat([take(pre + f"self_attn.{n}_proj.weight") for n in ("q", "k", "v")], dim=0))
                self.wo[l].copy_(take(pre + "self_attn.o_proj.weight"))
                g, u = take(pre + "mlp.gate_proj.weight"), take(pre + "mlp.up_proj.weight")
                self.wgu[l].copy_(torch.stack([g, u], dim=1).reshape(-1, g.shape[1]))
                self.wdown[l].copy_(take(pre + "mlp.down_proj.weight"))
                self.ln1[l].copy_(take(pre + "input_layernorm.weight"))
                self.ln2[l].copy_(take(pre + "post_attention_layernorm.weight"))
            self.norm.copy_(take("model.norm.weight"))
            self.lm_head.weight.copy_(take("lm_head.weight"))
        leftover = [k for k in sd if "rotary_emb" not in k]
        if strict and leftover:
            raise KeyError(f"unexpected keys in state dict: {leftover[:5]}")
        self._invalidate()
        return leftover

    @classmethod
    def from_pretrained(cls, path: str, torch_dtype: torch.dtype = torch.bfloat16, device="cuda") -> "LlamaForCausalLM":
        """A Hugging Face Llama checkpoint directory (config.json + safetensors / bin shards with the HF
        names), packed into the kernel layouts tensor by tensor (cmd/generate.py:55-63)."""
        import transformers

        cfg = transformers.LlamaConfig.from_pretrained(path)
        if getattr(cfg, "rope_theta", None) is None:
            cfg.rope_theta = float((getattr(cfg, "rope_parameters", None) or {}).get("rope_theta", 10000.0))
        model = cls(cfg).to(device=device, dtype=torch_dtype)
        ck = checkpoint.LazyCheckpoint(path)
        if "lm_head.weight" not in ck and getattr(cfg, "tie_word_embeddings", False):
            raise _lib.RedrafterError("checkpoints with tied input/output embeddings are not supported")
        model.load_state_dict(ck)
        return model

    def save_pretrained(self, path: str) -> None:
        """config.json + model.safetensors with the HF names."""
        checkpoint.save_directory(path, self.config, self.reference_state_dict())

    def reference_state_dict(self) -> Dict[str, torch.Tensor]:
        """The weights under the HF / reference names."""
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        sd = {"model.embed_tokens.weight": self.model.embed_tokens.weight.detach().clone()}
        for l in range(self.n_layers):
            pre = f"model.layers.{l}."
            q, k, v = torch.split(self.wqkv[l].detach(), [nh * hd, nkv * hd, nkv * hd], dim=0)
            sd[pre + "self_attn.q_proj.weight"], sd[pre + "self_attn.k_proj.weight"], sd[pre + "self_attn.v_proj.weight"] = q.clone(), k.clone(), v.clone()
            sd[pre + "self_attn.o_proj.weight"] = self.wo[l].detach().clone()
            gu = self.wgu[l].detach().reshape(-1, 2, self.wgu[l].shape[1])
            sd[pre + "mlp.gate_proj.weight"], sd[pre + "mlp.up_proj.weight"] = gu[:, 0].clone(), gu[:, 1].clone()
            sd[pre + "mlp.down_proj.weight"] = self.wdown[l].detach().clone()
            sd[pre + "input_layernorm.weight"] = self.ln1[l].detach().clone()
            sd[pre + "post_attention_layernorm.weight"] = self.ln2[l].detach().clone()
        sd["model.norm.weight"] = self.norm.detach().clone()
        sd["lm_head.weight"] = self.lm_head.weight.detach().clone()
        return sd

    def _apply(self, fn, *args, **kwargs):
        out = super()._apply(fn, *args, **kwargs)
        self._invalidate()
        return out

    def _invalidate(self):
        self._linears = None
        self._ws = {}
        self._ws_full = None
        self._ws_cap = (0, 0)
        self._rope = None
        self._head_ws = None
        self._drop_attn_plans()

    def _drop_attn_plans(self):
        plans = getattr(self, "_attn_plans", None)
        if plans:
            lib = _lib.load()
            for p in plans.values():
                lib.rd_attention_plan_destroy(p)
        self._attn_plans = {}

    def __del__(self):
        try:
            self._drop_attn_plans()
        except Exception:
            pass

    def _attention(self, code, q, kc, vc, attn, row_start, kv_begin, base_len, batch, m_max, max_new, max_kv, mode, tree_mask,
                   mask_words, dense_mask, dld_q, dld_b, st):
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        max_len = kc.shape[2]
        if self.dtype == torch.bfloat16 and hd == 128 and mode != _lib.ATTN_DENSE and mask_words <= 16:
            # tcgen05 path: TMA descriptors are tied to these exact buffers
            key = (q.data_ptr(), m_max, kc.data_ptr(), vc.data_ptr(), batch, max_len)
            plan = self._attn_plans.get(key)
            if plan is None:
                plan = _lib.load().rd_attention_plan_create(_lib.ptr(q), m_max, _lib.ptr(kc), _lib.ptr(vc), batch, nh, nkv, hd, max_len)
                if not plan:
                    raise _lib.RedrafterError("rd_attention_plan_create failed (TMA descriptor could not be encoded)")
                if len(self._attn_plans) >= 4 * self.n_layers:
                    self._drop_attn_plans()
                self._attn_plans[key] = plan
            shares = attention.key_range_shares(batch, nh, max_new, max_kv)
            if shares > 1:
                # few (row, head) chains and a long cache: several CTAs per chain, merged by a second kernel
                need = _lib.load().rd_attention_split_workspace_bytes(m_max, nh, shares)
                if self._attn_split_ws is None or self._attn_split_ws.numel() < need:
                    self._attn_split_ws = torch.empty(need, dtype=torch.uint8, device=q.device)
                _lib.call("rd_attention_tc_split", plan, _lib.ptr(attn), _lib.ptr(row_start), _lib.ptr(kv_begin), _lib.ptr(base_len),
                          max_new, mode, _lib.ptr(tree_mask), mask_words, shares, _lib.ptr(self._attn_split_ws),
                          self._attn_split_ws.numel(), _lib.ptr(self.gemm_status), st)
            else:
                _lib.call("rd_attention_tc", plan, _lib.ptr(attn), _lib.ptr(row_start), _lib.ptr(kv_begin), _lib.ptr(base_len),
                          max_new, mode, _lib.ptr(tree_mask), mask_words, _lib.ptr(self.gemm_status), st)
            return
        _lib.call("rd_attention", code, _lib.ptr(q), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(attn), _lib.ptr(row_start),
                  _lib.ptr(kv_begin), _lib.ptr(base_len), batch, nh, nkv, hd, max_len, max_new, max_kv, mode,
                  _lib.ptr(tree_mask), mask_words, _lib.ptr(dense_mask), dld_q, dld_b, st)

    # ----------------------------------------------------------------- kernels
    def _lin(self):
        if self._linears is None:
            self._linears = {
                "qkv": [_Linear(w) for w in self.wqkv],
                "o": [_Linear(w) for w in self.wo],
                "gu": [_Linear(w) for w in self.wgu],
                "down": [_Linear(w) for w in self.wdown],
                "head": _Linear(self.lm_head.weight),
            }
        return self._linears

    def _rope_tables(self, n_pos: int):
        if self._rope is None or self._rope[0].shape[0] < n_pos:
            self._rope = rope_tables(self.head_dim, max(n_pos, 2048), self.rope_theta, self.device)
        return self._rope

    def workspace(self, m_max: int, logit_rows: int) -> Dict[str, torch.Tensor]:
        """Activation buffers for m_max packed tokens and fp32 logits for logit_rows rows.  One
        grow-only set is kept (sized by the largest request seen); smaller requests get leading
        slices of it, so a process that serves prompts of many different sizes holds one set, not
        one per size.  When the set grows, the descriptors tied to the old buffers are dropped."""
        key = (m_max, logit_rows)
        ws = self._ws.get(key)
        if ws is not None:
            return ws
        H, dt, dev = self.config.hidden_size, self.dtype, self.device
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        cap_m, cap_l = self._ws_cap
        full = dict(self._ws_full or {})
        if m_max > cap_m:
            cap_m = m_max
            for name, width in (("h", H), ("xn", H), ("qkv", (nh + 2 * nkv) * hd), ("q", nh * hd), ("attn", nh * hd),
                                ("act", self.config.intermediate_size), ("hidden", H)):
                full[name] = torch.empty(cap_m, width, dtype=dt, device=dev)
            # folded RMS norm: per-token sums of squares by 128-feature slice
            full["ss"] = torch.empty(cap_m, ((H + 127) // 128 + 3) // 4 * 4, dtype=torch.float32, device=dev)
        if logit_rows > cap_l:
            cap_l = logit_rows
            full["logits"] = torch.empty(cap_l, self.config.vocab_size, dtype=torch.float32, device=dev)
        if (cap_m, cap_l) != self._ws_cap:
            self._ws_full, self._ws_cap = full, (cap_m, cap_l)
            self._ws = {}
            self._drop_plans()
        ws = {k: (v[:logit_rows] if k == "logits" else v[:m_max]) for k, v in full.items()}
        if len(self._ws) >= 16:
            self._ws.pop(next(iter(self._ws)))
        self._ws[key] = ws
        return ws

    def _drop_plans(self) -> None:
        """Forgets every TMA descriptor set (GEMM and attention plans); they are rebuilt on demand."""
        if self._linears is not None:
            for group in self._linears.values():
                for lin in (group if isinstance(group, list) else [group]):
                    lin.drop_plans()
        self._drop_attn_plans()

    def backbone(self, ws, cache_tensor: torch.Tensor, m_max: int, m_dev, tok_ids, tok_row, tok_pos, tok_slot, row_start,
                 kv_begin, base_len, batch: int, max_new: int, max_kv: int, mode: int, tree_mask=None, mask_words: int = 0,
                 dense_mask=None, n_pos: int = 4096) -> torch.Tensor:
        """Embedding + all decoder layers + final norm over m_max (or *m_dev) packed tokens.
        K/V of the tokens are written into cache_tensor [NL,2,B,nkv,max_len,hd].  Returns the
        post-norm hidden states ws["hidden"] (modeling_llama.py:207-237)."""
        code = _lib.dtype_code(self.dtype)
        lin = self._lin()
        H = self.config.hidden_size
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        max_len = cache_tensor.shape[4]
        cos, sin = self._rope_tables(n_pos)
        st = _lib.stream()
        md = _lib.ptr(m_dev)
        h, xn, qkv, q, attn, act = ws["h"], ws["xn"], ws["qkv"], ws["q"], ws["attn"], ws["act"]
        _lib.call("rd_embed_gather", code, _lib.ptr(self.model.embed_tokens.weight), _lib.ptr(tok_ids), _lib.ptr(h), m_max, md, H, st)
        dld_q = dense_mask.stride(1) if dense_mask is not None else 0
        dld_b = dense_mask.stride(0) if dense_mask is not None else 0
        fused_rope = (self.dtype == torch.bfloat16 and hd == 128 and H % 64 == 0 and xn.data_ptr() % 16 == 0
                      and os.environ.get("RD_FUSED_ROPE", "1") != "0")
        # RMS norms between the projections folded into them (RD_FUSED_NORM=1): o_proj / down_proj also write the
        # gamma-scaled row and its sums of squares, gate/up and the next layer's QKV apply 1 / rms in their epilogues;
        # the first layer's input norm and the final norm keep their own kernel.  Off unless asked for: it removes 63
        # launches of a 7B step, but the longer epilogues cost as much as the launches did.
        fused_norm = (fused_rope and H % 128 == 0 and h.data_ptr() % 16 == 0
                      and os.environ.get("RD_FUSED_NORM", "0") == "1")
        ss = ws["ss"] if fused_norm else None
        for l in range(self.n_layers):
            if not fused_norm or l == 0:
                _lib.call("rd_rmsnorm", code, _lib.ptr(h), _lib.ptr(self.ln1[l]), _lib.ptr(xn), m_max, md, H, self.eps, st)
            kc, vc = cache_tensor[l, 0], cache_tensor[l, 1]
            if fused_rope:
                # rotary embedding and the cache append ride on the projection's epilogue
                lin["qkv"][l].qkv_rope(xn, q, kc, vc, tok_row, tok_pos, tok_slot, cos, sin, nh, nkv, hd, m_dev, m_max,
                                       self.gemm_status, norm=(ss, H, self.eps) if fused_norm and l > 0 else None)
            else:
                lin["qkv"][l](xn, qkv, _lib.EPI_NONE, m_dev=m_dev, m_max=m_max, status=self.gemm_status)
                _lib.call("rd_rope_kv_write", code, _lib.ptr(qkv), _lib.ptr(q), _lib.ptr(kc), _lib.ptr(vc), _lib.ptr(tok_row),
                          _lib.ptr(tok_pos), _lib.ptr(tok_slot), _lib.ptr(cos), _lib.ptr(sin), cos.shape[0], m_max, md, nh, nkv,
                          hd, max_len, st)
            self._attention(code, q, kc, vc, attn, row_start, kv_begin, base_len, batch, m_max, max_new, max_kv, mode, tree_mask,
                            mask_words, dense_mask, dld_q, dld_b, st)
            if fused_norm:
                lin["o"][l].residual_with_norm(attn, h, h, self.ln2[l], xn, ss, m_dev, m_max, self.gemm_status)
                lin["gu"][l].swiglu_normed(xn, act, ss, H, self.eps, m_dev, m_max, self.gemm_status)
                if l + 1 < self.n_layers:
                    lin["down"][l].residual_with_norm(act, h, h, self.ln1[l + 1], xn, ss, m_dev, m_max, self.gemm_status)
                else:
                    lin["down"][l](act, h, _lib.EPI_RES, residual=h, m_dev=m_dev, m_max=m_max, status=self.gemm_status)
                continue
            lin["o"][l](attn, h, _lib.EPI_RES, residual=h, m_dev=m_dev, m_max=m_max, status=self.gemm_status)
            _lib.call("rd_rmsnorm", code, _lib.ptr(h), _lib.ptr(self.ln2[l]), _lib.ptr(xn), m_max, md, H, self.eps, st)
            lin["gu"][l](xn, act, _lib.EPI_SWIGLU, m_dev=m_dev, m_max=m_max, status=self.gemm_status)
            lin["down"][l](act, h, _lib.EPI_RES, residual=h, m_dev=m_dev, m_max=m_max, status=self.gemm_status)
        _lib.call("rd_rmsnorm", code, _lib.ptr(h), _lib.ptr(self.norm), _lib.ptr(ws["hidden"]), m_max, md, H, self.eps, st)
        return ws["hidden"]

    def lm_logits(self, hidden_rows: torch.Tensor, logits: torch.Tensor, m_dev=None) -> torch.Tensor:
        """fp32 logits of the given hidden rows (modeling_llama.py:272)."""
        self._lin()["head"](hidden_rows, logits, _lib.EPI_NONE, m_dev=m_dev, status=self.gemm_status)
        return logits

    def fused_head_ok(self) -> bool:
        """The LM head can run with the arg-max or the slice maxima in its epilogue (bf16 tensor-core path,
        vocabulary a multiple of 32)."""
        return (self.dtype == torch.bfloat16 and self.config.hidden_size % 64 == 0 and self.config.vocab_size % 32 == 0
                and os.environ.get("RD_FUSED_HEAD", "1") != "0")

    def _head_scratch(self, rows: int) -> torch.Tensor:
        """fp32 [vocab/32, rows rounded up to 32] scratch of the fused LM-head epilogues, grow-only."""
        slices = (self.config.vocab_size + 31) // 32
        ld = (rows + 31) // 32 * 32
        if self._head_ws is None or self._head_ws.shape[1] < ld:
            self._head_ws = torch.empty(2 * slices, ld, dtype=torch.float32, device=self.device)
        return self._head_ws

    def lm_argmax(self, hidden_rows: torch.Tensor, out32: torch.Tensor, m_dev=None) -> None:
        """Greedy tokens of the given hidden rows, int32, without writing the logits (modeling_llama.py:272 +
        recurrent_drafting.py:52)."""
        rows = hidden_rows.shape[0]
        ws = self._head_scratch(rows)
        need = _lib.load().rd_gemm_argmax_workspace_bytes(rows, self.config.vocab_size)
        flat = ws.view(-1).view(torch.uint8)
        assert flat.numel() >= need
        self._lin()["head"].argmax(hidden_rows, out32, flat, m_dev, rows, self.gemm_status)

    def lm_logits_with_slice_max(self, hidden_rows: torch.Tensor, logits: torch.Tensor, m_dev=None) -> Optional[torch.Tensor]:
        """lm_logits() that also returns the [vocab/32, rows'] slice maxima for rd_vocab_topk_sliced, or None
        (plain logits computed) when the fused epilogue does not apply."""
        rows = hidden_rows.shape[0]
        if self.fused_head_ok():
            smax = self._head_scratch(rows)[: self.config.vocab_size // 32]
            if self._lin()["head"].with_slice_max(hidden_rows, logits, smax, m_dev=m_dev, status=self.gemm_status):
                return smax
        self.lm_logits(hidden_rows, logits, m_dev=m_dev)
        return None

    # ----------------------------------------------------------------- reference forward
    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor, attention_mask: torch.Tensor, position_ids: torch.Tensor,
                past_key_values) -> CausalLMOutput:
        """The reference call (modeling_llama.py:255-276): padded (batch, q_len) ids, explicit bool
        mask (batch, q_len, kv_len), positions, cache views; K/V of the q_len tokens are appended to
        every view."""
        B, q_len = input_ids.shape
        dev = input_ids.device
        view0 = past_key_values[0][0]
        assert isinstance(view0, kv_cache.View)
        S = view0.length
        cache_tensor = view0._cache
        assert attention_mask.shape == (B, q_len, S + q_len), (attention_mask.shape, (B, q_len, S + q_len))
        assert S + q_len <= cache_tensor.shape[4]
        M = B * q_len
        i32 = dict(dtype=torch.int32, device=dev)
        tok_row = torch.arange(B, **i32).repeat_interleave(q_len)
        tok_slot = (S + torch.arange(q_len, **i32)).repeat(B)
        tok_pos = position_ids.reshape(-1).clamp(min=0).to(torch.int32)
        row_start = torch.arange(B + 1, **i32) * q_len
        kv_begin = torch.zeros(B, **i32)
        base_len = torch.full((B,), S, **i32)
        dense = attention_mask.to(torch.uint8).contiguous()
        ws = self.workspace(M, M)
        n_pos = max(4096, int(S + q_len) + 1)
        hidden = self.backbone(ws, cache_tensor, M, None, input_ids.reshape(-1).contiguous(), tok_row, tok_pos, tok_slot,
                               row_start, kv_begin, base_len, B, q_len, S + q_len, _lib.ATTN_DENSE, dense_mask=dense,
                               n_pos=n_pos)
        logits = self.lm_logits(hidden, ws["logits"])
        for k, v in past_key_values:
            k.length = v.length = S + q_len
        V = self.config.vocab_size
        return CausalLMOutput(logits=logits.view(B, q_len, V).clone(), hidden_states=hidden.view(B, q_len, -1).clone())
