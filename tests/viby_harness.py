"""A from-scratch functional Viby forward for the whole-model configuration (config 4): 18
blocks of RMSNorm -> Canon A -> attention (Canon B on q|k|v) -> RMSNorm -> Canon C -> SwiGLU MLP
(Canon D on gate|up), tied embedding / LM head.  TEST INFRASTRUCTURE: it exists so that the Canon
kernels can be exercised inside a full forward on a machine that has no copy of the reference.

Written from the structure of the reference (model/model.py:692-926 attention with causal,
key-padding and sliding-window masks and a per-head sink logit; :950-976 MLP; :1006-1068 block;
:1115-1157 model; :116-122, :185-197 RoPE) and checked against it: tests/golden/viby_tiny.npz holds
a tiny reference model's weights, inputs and logits (generator: tests/golden/make_model_golden.py),
and tests/test_model_harness.py requires this harness in ``canon="fallback"`` mode to reproduce them.

Canon modes:
  "fallback"  the reference's PyTorch branch (masked residual, 8-column state), via the oracle
  "torch"     the reference's CUDA-branch semantics (unmasked prefill residual, masked decode
              residual, kernel_size-column state) with torch ops on the tensor's own device
  "kernel"    the same semantics through viby_model_b200 (fused mask / residual / final state)
  "kernel_plain"  the kernels called exactly as the reference's CUDA branch calls them
              (model/model.py:454-491 and 299-313): through the drop-in module ``causal_conv1d``, keyword
              arguments ``x=, weight=, bias=, activation=, seq_idx=None`` / ``x=, conv_state=, ...``, with
              the mask multiply, the state seeding and the residual left to torch ops around the call
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F


def rms_norm(x, weight, eps):
    return F.rms_norm(x, (x.shape[-1],), weight, eps)


def rope_tables(head_dim: int, end: int, theta: float, device, dtype=torch.float32):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device).float() / head_dim))
    ang = torch.outer(torch.arange(end, device=device).float(), inv)
    return torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)


def rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


class VibyHarness:
    def __init__(self, cfg: Dict, params: Dict[str, torch.Tensor], canon: str = "kernel"):
        self.cfg = cfg
        self.p = params
        self.canon = canon
        self.hd = cfg["hidden_size"] // cfg["num_attention_heads"]
        dev = params["model.embed_tokens.weight"].device
        self.cos, self.sin = rope_tables(self.hd, cfg.get("max_positions", 4096), cfg["rope_theta"], dev)
        # set to a list to record (name, layer, x, mask, out, conv term or None) of every prefill Canon call
        self.canon_inputs = None

    # ---- Canon layer ------------------------------------------------------------------------------
    def _canon(self, x, name, layer, mask, cache):
        w = self.p[f"model.layers.{layer}.{name}.weight"].squeeze(1)
        b = self.p.get(f"model.layers.{layer}.{name}.bias_param")
        act = self.cfg["canon_activation"]
        K = w.shape[1]
        key = (layer, name)
        B, T, D = x.shape
        if self.canon == "fallback":
            from oracle import canon_oracle as O

            state = cache["canon"].get(key) if cache is not None else None
            y, state = O.canon_layer_ref(x, w, b, act, attention_mask=mask, conv_state=state,
                                         use_cache=cache is not None, native_dtype=True)
            if cache is not None:
                cache["canon"][key] = state
            return y
        decode = cache is not None and T == 1
        if decode:
            xt = x.squeeze(1)
            if mask is not None:
                xt = xt * mask[:, -1].unsqueeze(-1).to(xt.dtype)
            state = cache["canon"].get(key)
            if state is None or state.shape[-1] != K:
                state = torch.zeros(B, D, K, dtype=x.dtype, device=x.device)
                cache["canon"][key] = state
            if self.canon == "kernel":
                import viby_model_b200 as V

                y = V.causal_conv1d_update(xt, state, w, b, activation="silu" if act else None)
            elif self.canon == "kernel_plain":
                import causal_conv1d as CC

                y = CC.causal_conv1d_update(x=xt, conv_state=state, weight=w, bias=b,
                                            activation="silu" if act else None)  # model/model.py:305-311
            else:
                cat = torch.cat([state, xt.unsqueeze(-1)], -1)
                y = (cat[..., -K:].float() * w.float()).sum(-1)
                if b is not None:
                    y = y + b.float()
                if act:
                    y = F.silu(y)
                y = y.to(x.dtype)
                state.copy_(cat[..., -K:])
            return (xt + y).unsqueeze(1)
        m = None
        if mask is not None:
            m = mask[:, -T:] if mask.shape[1] >= T else torch.cat(
                [mask, torch.ones(B, T - mask.shape[1], dtype=mask.dtype, device=mask.device)], 1)
        if self.canon == "kernel":
            import viby_model_b200 as V

            res = V.causal_conv1d_fn(x.transpose(1, 2), w, b, activation="silu" if act else None, attention_mask=m,
                                     residual=True, return_final_states=cache is not None, state_len=K)
            if cache is not None:
                y, cache["canon"][key] = res
            else:
                y = res
            out = y.transpose(1, 2)
        elif self.canon == "kernel_plain":
            import causal_conv1d as CC

            xm = x * m.unsqueeze(-1).to(x.dtype) if m is not None else x            # model/model.py:454-457
            y = CC.causal_conv1d_fn(x=xm.transpose(1, 2), weight=w, bias=b, activation="silu" if act else None,
                                    seq_idx=None)                                    # :460-466
            conv_term = y.transpose(1, 2)
            out = x + conv_term                                                       # :491
            if cache is not None:                                                     # :470-489
                st = torch.zeros(B, D, K, dtype=x.dtype, device=x.device)
                n = min(T, K)
                st[..., K - n:] = xm.transpose(1, 2)[..., T - n:]
                cache["canon"][key] = st
            if self.canon_inputs is not None:
                self.canon_inputs.append((name, layer, x, m, out, conv_term))
            return out
        else:
            xm = x * m.unsqueeze(-1).to(x.dtype) if m is not None else x
            conv = F.conv1d(F.pad(xm.transpose(1, 2).float(), (K - 1, 0)), w.float().unsqueeze(1),
                            b.float() if b is not None else None, groups=D)
            if act:
                conv = F.silu(conv)
            out = x + conv.to(x.dtype).transpose(1, 2)
            if cache is not None:
                st = torch.zeros(B, D, K, dtype=x.dtype, device=x.device)
                n = min(T, K)
                st[..., K - n:] = xm.transpose(1, 2)[..., T - n:]
                cache["canon"][key] = st
        if self.canon_inputs is not None:
            self.canon_inputs.append((name, layer, x, m, out, None))
        return out

    # ---- attention ----------------------------------------------------------------------------------
    def _attention(self, x, layer, mask, cache, start):
        c = self.cfg
        H, KV, hd = c["num_attention_heads"], c["num_key_value_heads"], self.hd
        B, T, _ = x.shape
        pre = f"model.layers.{layer}.self_attn."
        q = F.linear(x, self.p[pre + "q_proj.weight"])
        k = F.linear(x, self.p[pre + "k_proj.weight"])
        v = F.linear(x, self.p[pre + "v_proj.weight"])
        qkv = self._canon(torch.cat([q, k, v], -1), "self_attn.canon_b", layer, mask, cache)
        q, k, v = qkv.split([H * hd, KV * hd, KV * hd], -1)
        q = q.reshape(B, T, H, hd)
        k = k.reshape(B, T, KV, hd)
        v = v.reshape(B, T, KV, hd)
        cos = self.cos[start:start + T].to(x.dtype).unsqueeze(1)
        sin = self.sin[start:start + T].to(x.dtype).unsqueeze(1)
        q = q * cos + rotate_half(q) * sin
        k = k * cos + rotate_half(k) * sin
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        if cache is not None:
            if layer in cache["k"]:
                k = torch.cat([cache["k"][layer], k], 2)
                v = torch.cat([cache["v"][layer], v], 2)
            cache["k"][layer], cache["v"][layer] = k, v
        rep = H // KV
        kk = k.repeat_interleave(rep, 1)
        vv = v.repeat_interleave(rep, 1)
        scores = torch.einsum("bhqd,bhkd->bhqk", q, kk) * torch.tensor(1.0 / math.sqrt(hd), dtype=q.dtype, device=q.device)
        Tk = scores.shape[-1]
        past = Tk - T
        neg = torch.finfo(scores.dtype).min
        qa = torch.arange(T, device=x.device) + past
        ka = torch.arange(Tk, device=x.device)
        scores = scores.masked_fill(ka[None, :] > qa[:, None], neg)
        if mask is not None:
            am = mask
            if am.shape[1] < Tk:
                am = torch.cat([am, torch.ones(B, Tk - am.shape[1], dtype=am.dtype, device=am.device)], 1)
            elif am.shape[1] > Tk:
                am = am[:, -Tk:]
            scores = scores.masked_fill((am == 0)[:, None, None, :], neg)
        win = 0 if (layer + 1) % 6 == 0 else c["sliding_window"]
        if win and win > 0:
            scores = scores.masked_fill(~(ka[None, :] >= (qa[:, None] - win)), neg)
        sink = self.p[pre + "sinks"].view(1, H, 1, 1).to(scores.dtype).expand(B, -1, T, 1)
        w = F.softmax(torch.cat([scores, sink], -1), -1)[..., :-1]
        o = torch.einsum("bhqk,bhkd->bhqd", w, vv).transpose(1, 2).reshape(B, T, H * hd)
        return F.linear(o, self.p[pre + "o_proj.weight"])

    def _mlp(self, x, layer, mask, cache):
        pre = f"model.layers.{layer}.mlp."
        g = F.linear(x, self.p[pre + "gate_proj.weight"])
        u = F.linear(x, self.p[pre + "up_proj.weight"])
        gu = self._canon(torch.cat([g, u], -1), "mlp.canon_d", layer, mask, cache)
        g, u = gu[..., : g.shape[-1]], gu[..., g.shape[-1]:]
        return F.linear(F.silu(g) * u, self.p[pre + "down_proj.weight"])

    def new_cache(self):
        return {"k": {}, "v": {}, "canon": {}, "len": 0}

    @torch.no_grad()
    def forward(self, ids, attention_mask: Optional[torch.Tensor] = None, cache: Optional[dict] = None):
        c = self.cfg
        eps = c["rms_norm_eps"]
        start = cache["len"] if cache is not None else 0
        h = F.embedding(ids, self.p["model.embed_tokens.weight"])
        for layer in range(c["num_hidden_layers"]):
            pre = f"model.layers.{layer}."
            n = rms_norm(h, self.p[pre + "input_layernorm.weight"], eps)
            n = self._canon(n, "canon_a", layer, attention_mask, cache)
            h = h + self._attention(n, layer, attention_mask, cache, start)
            n = rms_norm(h, self.p[pre + "post_attention_layernorm.weight"], eps)
            n = self._canon(n, "canon_c", layer, attention_mask, cache)
            h = h + self._mlp(n, layer, attention_mask, cache)
        if cache is not None:
            cache["len"] = start + ids.shape[1]
        h = rms_norm(h, self.p["model.norm.weight"], eps)
        return F.linear(h, self.p["model.embed_tokens.weight"])


def random_params(cfg: Dict, seed: int, dtype, device, std: float = 0.02) -> Dict[str, torch.Tensor]:
    """All parameters ~ N(0, std), as the whole-model configuration specifies (norm weights too)."""
    g = torch.Generator().manual_seed(seed)
    Hs, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    H, KV = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = Hs // H
    K = cfg["canon_kernel"]

    def t(*shape):
        return (torch.randn(*shape, generator=g) * std).to(dtype).to(device)

    p = {"model.embed_tokens.weight": t(V, Hs), "model.norm.weight": t(Hs)}
    for layer in range(cfg["num_hidden_layers"]):
        pre = f"model.layers.{layer}."
        p[pre + "input_layernorm.weight"] = t(Hs)
        p[pre + "post_attention_layernorm.weight"] = t(Hs)
        p[pre + "self_attn.q_proj.weight"] = t(H * hd, Hs)
        p[pre + "self_attn.k_proj.weight"] = t(KV * hd, Hs)
        p[pre + "self_attn.v_proj.weight"] = t(KV * hd, Hs)
        p[pre + "self_attn.o_proj.weight"] = t(Hs, H * hd)
        p[pre + "self_attn.sinks"] = t(H)
        p[pre + "mlp.gate_proj.weight"] = t(I, Hs)
        p[pre + "mlp.up_proj.weight"] = t(I, Hs)
        p[pre + "mlp.down_proj.weight"] = t(Hs, I)
        for name, dim in (("canon_a", Hs), ("self_attn.canon_b", (H + 2 * KV) * hd), ("canon_c", Hs),
                          ("mlp.canon_d", 2 * I)):
            p[pre + name + ".weight"] = t(dim, 1, K)
            if cfg["canon_bias"]:
                p[pre + name + ".bias_param"] = t(dim)
    return p
