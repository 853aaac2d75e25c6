"""Hybrid sequence models (decoder-only language models built from state-space, gated-linear-attention, delta-rule, chunk-local
attention, retention, latent-attention and sliding-window attention mixers, in post-norm blocks, pre-norm blocks on several
residual streams, parallel blocks or blocks normed on the sublayer's output, with dense or routed feed-forwards) behind the same surface as the video-language engine: `from_pretrained`, `generate`, a cache object that
callers pass back, greedy token selection in the library's sampling kernel.

    model = SeqLMForCausalLM.from_pretrained(path, torch_dtype="bfloat16", device_map="cuda")
    out = model.generate(input_ids, max_new_tokens=16)            # out.sequences, out.past_key_values
    logits = model.forward_step([(cache, ids)], [[0, 2]])         # teacher-forced step: logits of chosen rows

Everything numeric runs in the native library (csrc/seq_model.cu sequences one step; linear_any.cu / gemm_tcgen05.cu,
recurrent.cu, attn_local.cu, attn_latent.cu, moe.cu, rowops.cu hold the kernels); this file is host orchestration: weight layout, state slots and
pages, step bookkeeping, CUDA-graph replay of the decode step. There is no CPU or eager fallback.

Two storage types: bf16 (weights, activations and K/V pages in bf16; the residual stream, norms, scores, recurrent state
and everything entering a recurrence in fp32) and fp32 (everything fp32, plain FMAs).
"""
from __future__ import annotations

import ctypes as C
import json
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _cabi
from .config import SeqModelConfig
from .engine import GenerateOutput
from .kv_cache import PAGE_SIZE, SeqCache, SeqStatePool


def _dtype_of(torch_dtype) -> torch.dtype:
    if torch_dtype in ("auto", None, torch.bfloat16, "bfloat16", "bf16"):
        return torch.bfloat16
    if torch_dtype in (torch.float32, "float32", "fp32", "float"):
        return torch.float32
    raise NotImplementedError(f"torch_dtype={torch_dtype!r}: the hybrid sequence models run in bfloat16 or float32")


class SeqWeights:
    """Device tensors in the layout the library reads: fused input projections per mixer, fp32 norms / biases / per-head
    parameters, matrices in the storage type."""

    def __init__(self, cfg: SeqModelConfig, tensors, dtype: torch.dtype, device):
        t: Dict[str, torch.Tensor] = dict(tensors)
        self.dtype = dtype
        used = set()

        def get(name):
            if name not in t:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            return t[name]

        def mat(*names):   # rows of several [out, in] matrices stacked into one; row count padded to 8 with zero rows
            m = torch.cat([get(n).to(torch.float32) for n in names], 0)
            if m.shape[0] % 8:
                m = torch.cat([m, torch.zeros((-m.shape[0]) % 8, m.shape[1], dtype=m.dtype, device=m.device)], 0)
            return m.to(device=device, dtype=dtype).contiguous()

        def shape(name):
            return tuple(get(name).shape)

        def f32(x):
            return x.to(device=device, dtype=torch.float32).contiguous()

        def norm_w(name):   # layer norms whose weights are stored around zero are applied as 1 + w (summed in fp32)
            if cfg.norm_scalar:     # one number for all coordinates: the kernels read a weight per column
                if get(name).numel() != 1:
                    raise ValueError(f"{name} is not a single number")
                return f32(get(name).to(torch.float32).reshape(1).expand(cfg.width))
            return f32(get(name).to(torch.float32) + cfg.norm_offset) if cfg.norm_offset else f32(get(name))

        def segments(names, pad_cols=None):   # blocks of rows stacked with every block's start at a multiple of 8 rows
            parts = []
            for n in names:
                m = get(n).to(torch.float32)
                m = m.reshape(m.shape[0], -1)
                parts.append(m)
                if m.shape[0] % 8:
                    parts.append(torch.zeros((-m.shape[0]) % 8, m.shape[1], dtype=m.dtype, device=m.device))
            return torch.cat(parts, 0)

        def check(name, want):
            if shape(name) != tuple(want):
                raise ValueError(f"{name} has shape {shape(name)}, config.json implies {tuple(want)}")

        def rotary(rot):
            freq, mag = rot.frequencies()
            return torch.tensor(freq, dtype=torch.float64).to(torch.float32).to(device), float(mag)

        dyt = cfg.norm == "dyt"

        def norm_extra(name):   # a Dynamic-Tanh norm keeps a bias vector and a scalar beside its weight
            if not dyt:
                return None, 0.0
            check(name + ".b", (W,))
            if get(name + ".alpha").numel() != 1:
                raise ValueError(f"{name}.alpha is not a scalar")
            return f32(get(name + ".b")), float(get(name + ".alpha").to(torch.float32).reshape(-1)[0])

        W = cfg.width
        self.embed = mat("embed")
        self.head = mat("head")
        self.final_norm = norm_w("final.norm")
        self.final_norm_bias, self.final_norm_alpha = norm_extra("final.norm")
        if shape("embed") != (cfg.vocab, W) or shape("head") != (cfg.vocab, W):
            raise ValueError("embed / head do not have the shape [vocab, width] of config.json")
        self.inv_freq = None
        if cfg.positions == "sinusoid":
            i2 = torch.arange(0, W, 2, dtype=torch.float32)
            self.inv_freq = torch.pow(torch.tensor(10000.0, dtype=torch.float32), -i2 / W).to(device)
        hc = cfg.block == "prenorm_hc"
        self.layers: List[dict] = []
        for i, L in enumerate(cfg.layers):
            if L.weights_of >= 0:            # the layer runs with another layer's tensors (its cache and state are its own):
                self.layers.append(None)     # filled in below, once every owner is built
                continue
            p = f"l{i}."
            w = {"norm1": norm_w(p + "norm1")}
            w["norm1_bias"], w["norm1_alpha"] = norm_extra(p + "norm1")
            if hc:
                n = cfg.streams
                for q in ("hc1", "hc2") if (L.ff or L.moe) else ("hc1",):
                    a = p + q + "."
                    check(a + "in", (n,)), check(a + "out", (n,)), check(a + "mix", (n, n))
                    w[q] = f32(torch.cat([get(a + "in").float().reshape(-1), get(a + "out").float().reshape(-1),
                                          get(a + "mix").float().reshape(-1)]))
            if cfg.canon_taps:
                check(p + "canon1", (W, cfg.canon_taps))
                w["canon"] = f32(get(p + "canon1"))
            if L.type == "channel_delta":
                dl, m = L.delta, p + "mix."
                nk, nv = dl.kv_heads * dl.dim, dl.heads * dl.vdim
                dl.rank_a, dl.rank_g = int(shape(m + "a1")[0]), int(shape(m + "g1")[0])
                check(m + "q", (nk, W)), check(m + "k", (nk, W)), check(m + "v", (nv, W)), check(m + "b", (dl.heads, W))
                check(m + "q.conv", (nk, dl.conv)), check(m + "k.conv", (nk, dl.conv)), check(m + "v.conv", (nv, dl.conv))
                check(m + "a1", (dl.rank_a, W)), check(m + "a2", (dl.heads * dl.dim, dl.rank_a)), check(m + "dt_bias", (dl.heads * dl.dim,))
                check(m + "A_log", (dl.heads,)), check(m + "g1", (dl.rank_g, W)), check(m + "g2", (nv, dl.rank_g))
                check(m + "norm", (dl.vdim,)), check(m + "o", (W, nv))
                # one input projection [q | k | v | beta | decay-down | gate-down], every block starting at a multiple of 8 rows; the
                # convolution's taps follow the q, k, v blocks (zero taps on the padding channels)
                w["d_in"] = segments([m + "q", m + "k", m + "v", m + "b", m + "a1", m + "g1"]).to(device=device, dtype=dtype).contiguous()
                w["d_conv_w"] = f32(segments([m + "q.conv", m + "k.conv", m + "v.conv"]))
                w["d_a_up"], w["d_g_up"], w["d_out"] = mat(m + "a2"), mat(m + "g2"), mat(m + "o")
                w["d_dt_bias"], w["d_a_log"], w["d_norm"] = f32(get(m + "dt_bias")), f32(get(m + "A_log")), f32(get(m + "norm"))
            elif L.type == "retention":
                rt, m = L.retention, p + "mix."
                check(m + "q", (rt.heads * rt.dim, W)), check(m + "k", (rt.heads * rt.dim, W))
                check(m + "v", (rt.heads * rt.vdim, W)), check(m + "g", (rt.heads * rt.vdim, W)), check(m + "o", (W, rt.heads * rt.vdim))
                w["t_in"] = mat(m + "q", m + "k", m + "v", m + "g")
                w["t_out"] = mat(m + "o")
                w["t_log_decay"] = torch.log(torch.tensor(rt.decay, dtype=torch.float64)).to(torch.float32).to(device)
                w["t_norm"] = torch.ones(rt.vdim, dtype=torch.float32, device=device)
                if rt.rot.dims:
                    w["rot_freq"], w["rot_mag"] = rotary(rt.rot)
            elif L.type == "latent_attention":
                a, m = L.latent, p + "mix."
                check(m + "uk", (a.heads * a.dim, a.kv_rank)), check(m + "uv", (a.heads * a.vdim, a.kv_rank))
                check(m + "o", (W, a.heads * a.vdim))
                if a.q_rank or (m + "dq") in t:      # queries through a latent of their own: [down | norm | up]
                    a.q_rank = int(shape(m + "dq")[0])
                    check(m + "dq", (a.q_rank, W)), check(m + "dq.norm", (a.q_rank,)), check(m + "uq", (a.heads * (a.dim + a.rot_dim), a.q_rank))
                    rows = [m + "dq"]
                    w["a_q_norm"], w["a_uq"] = f32(get(m + "dq.norm")), mat(m + "uq")
                else:
                    check(m + "q", (a.heads * (a.dim + a.rot_dim), W))
                    rows = [m + "q"]
                if a.kv_from < 0:
                    check(m + "dkv", (a.kv_rank + a.rot_dim, W)), check(m + "dkv.norm", (a.kv_rank,))
                    rows.append(m + "dkv")
                    w["a_latent_norm"] = f32(get(m + "dkv.norm"))
                if a.gate:
                    check(m + "g", (a.heads, W))
                    rows.append(m + "g")
                w["a_in"] = mat(*rows)
                # query absorption reads each head's key up-projection transposed: [heads][rank][dim]
                w["a_uk_t"] = get(m + "uk").to(torch.float32).reshape(a.heads, a.dim, a.kv_rank).transpose(1, 2) \
                    .contiguous().to(device=device, dtype=dtype)
                w["a_uv"] = mat(m + "uv")
                if a.sink:
                    check(m + "sink", (a.heads,))
                    w["a_sink"] = f32(get(m + "sink"))
                w["a_out"] = mat(m + "o")
                w["rot_freq"], w["rot_mag"] = rotary(a.rot)
            elif L.type == "attention":
                a, m = L.attn, p + "mix."
                check(m + "q", (a.heads * a.dim, W)), check(m + "k", (a.kv_heads * a.dim, W)), check(m + "o", (W, a.heads * a.vdim))
                if not a.unit_norm:
                    check(m + "q.norm", (a.dim,)), check(m + "k.norm", (a.dim,))
                    w["m_qnorm"], w["m_knorm"] = f32(get(m + "q.norm")), f32(get(m + "k.norm"))
                if a.temp:
                    check(m + "temp", (a.heads,))
                    w["m_temp"] = f32(get(m + "temp"))
                if a.v_mix:      # the first such layer keeps its values for the later ones, whose `vmix` blends them in
                    first = next(j for j, x in enumerate(cfg.layers) if x.type == "attention" and x.attn.v_mix)
                    if get(m + "vmix").numel() != 1:
                        raise ValueError(f"{m}vmix is not a single number")
                    w["m_vmix_role"] = 1 if first == i else 2
                    w["m_vmix"] = float(get(m + "vmix").to(torch.float32).reshape(-1)[0])
                rows = [m + "q", m + "k"]
                if not a.value_keys:
                    check(m + "v", (a.kv_heads * a.vdim, W))
                    rows.append(m + "v")
                if a.gate != "none":
                    check(m + "g", (a.gate_rows, W))
                    rows.append(m + "g")
                w["m_in"] = mat(*rows)
                w["m_out"] = mat(m + "o")
                if a.rot.dims:
                    w["rot_freq"], w["rot_mag"] = rotary(a.rot)
            elif L.type == "mamba2":
                s = L.ssd
                m = p + "mix."
                w["s_in"] = mat(m + "in")
                if shape(m + "in") != (s.proj_rows, W):
                    raise ValueError(f"{m}in has shape {shape(m + 'in')}, config.json implies {(s.proj_rows, W)}")
                w["s_conv_w"] = f32(get(m + "conv"))
                if w["s_conv_w"].shape != (s.conv_channels, s.conv):
                    raise ValueError(f"{m}conv has shape {tuple(w['s_conv_w'].shape)}, expected {(s.conv_channels, s.conv)}")
                w["s_conv_b"] = f32(get(m + "conv.b"))
                w["s_dt_bias"] = f32(get(m + "dt_bias"))
                w["s_a_log"] = f32(get(m + "A_log"))
                w["s_skip"] = f32(get(m + "D"))
                w["s_norm"] = f32(get(m + "norm"))
                w["s_out"] = mat(m + "o")
            else:
                l, r = L.left, L.right
                a, b = p + "mix.left.", p + "mix.right."
                w["l_in"] = mat(a + "q", a + "k", a + "v", a + "g")
                qb = get(a + "q.b")
                bias = torch.cat([qb.float(), get(a + "k.b").float(), get(a + "v.b").float(),
                                  torch.zeros(l.heads + (-(shape(a + "q")[0] + shape(a + "k")[0] + shape(a + "v")[0] + l.heads)) % 8,
                                              device=qb.device)])
                w["l_in_bias"] = f32(bias)
                w["l_in_bias_st"] = bias.to(device=device, dtype=dtype).contiguous()
                if (shape(a + "q")[0], shape(a + "k")[0], shape(a + "v")[0], shape(a + "g")[0]) != \
                        (l.heads * l.dim, l.kv_heads * l.dim, l.kv_heads * l.vdim, l.heads):
                    raise ValueError(f"layer {i}: left projections do not match config.json")
                w["l_qnorm"] = f32(get(a + "q.norm"))
                w["l_knorm"] = f32(get(a + "k.norm"))
                w["l_out"] = mat(a + "o")
                w["l_branch_norm"] = f32(get(a + "out"))
                r.rank = int(get(b + "a1").shape[0])
                w["r_in"] = mat(b + "q", b + "k", b + "v", b + "g", b + "a1")
                if (shape(b + "q")[0], shape(b + "k")[0], shape(b + "v")[0], shape(b + "g")[0]) != \
                        (r.heads * r.dim, r.heads * r.dim, r.heads * r.vdim, r.heads * r.vdim):
                    raise ValueError(f"layer {i}: right projections do not match config.json")
                w["r_decay_up"] = mat(b + "a2")
                w["r_decay_bias"] = f32(get(b + "a2.b"))
                w["r_norm"] = f32(get(b + "norm"))
                w["r_out"] = mat(b + "o")
                w["r_branch_norm"] = f32(get(b + "out"))
            par = cfg.block == "parallel"      # one norm per layer: the feed-forward reads the mixer's input
            if L.moe:
                e, m = L.moe, p + "mlp."
                if not par:
                    w["norm2"] = norm_w(p + "norm2")
                for j in range(e.experts):
                    check(f"{m}e{j}.up", (e.ff, W)), check(f"{m}e{j}.down", (W, e.ff))
                check(m + "router", (e.outputs, W))
                if e.router != "topk_softmax":
                    check(m + "correction", (e.outputs,))
                if e.act in ("clamp_glu", "silu_glu"):
                    # each expert's gate and up rows in one matrix, so that one product per expert list yields both. Widths that
                    # are multiples of 16 interleave them in groups of 16 rows (the layout whose activation the tensor-core
                    # product's epilogue forms from neighbouring accumulator columns); other widths keep [gate | up].
                    for j in range(e.experts):
                        check(f"{m}e{j}.gate", (e.ff, W))
                    w["e_up_il16"] = int(e.ff % 16 == 0)

                    def gate_up(j):
                        g, u = get(f"{m}e{j}.gate"), get(f"{m}e{j}.up")
                        if not w["e_up_il16"]:
                            return torch.cat([g, u], 0)
                        return torch.stack([g.view(e.ff // 16, 16, W), u.view(e.ff // 16, 16, W)], 1).reshape(2 * e.ff, W)

                    w["e_up"] = torch.stack([gate_up(j) for j in range(e.experts)]).to(device=device, dtype=dtype).contiguous()
                else:
                    w["e_up"] = torch.stack([get(f"{m}e{j}.up") for j in range(e.experts)]).to(device=device, dtype=dtype).contiguous()
                w["e_down"] = torch.stack([get(f"{m}e{j}.down") for j in range(e.experts)]).to(device=device, dtype=dtype).contiguous()
                if e.router != "topk_softmax":
                    w["e_correction"] = f32(get(m + "correction"))
                if e.shared_ff:
                    check(m + "shared.up", (e.shared_ff, W)), check(m + "shared.down", (W, e.shared_ff)), check(m + "shared.sg", (1, W))
                    w["e_router"] = mat(m + "router", m + "shared.sg")     # the shared gate's logit is one more router row
                    w["e_shared_up"], w["e_shared_down"] = mat(m + "shared.up"), mat(m + "shared.down")
                else:
                    w["e_router"] = mat(m + "router")
            elif L.ff:
                if not par:
                    w["norm2"] = norm_w(p + "norm2")
                check(p + "mlp.up", (L.ff, W)), check(p + "mlp.down", (W, L.ff))
                if cfg.dense == "mlp":
                    w["ff_in"] = mat(p + "mlp.up")
                else:
                    check(p + "mlp.gate", (L.ff, W))
                    w["ff_in"] = mat(p + "mlp.gate", p + "mlp.up")
                w["ff_out"] = mat(p + "mlp.down")
            self.layers.append(w)
        for i, L in enumerate(cfg.layers):
            if L.weights_of >= 0:
                self.layers[i] = self.layers[L.weights_of]
        self.unused = sorted(set(t) - used)

    def nbytes(self) -> int:
        n = sum(x.numel() * x.element_size() for x in (self.embed, self.head, self.final_norm))
        own = {id(w): w for w in self.layers}.values()      # layers that share tensors count once
        return n + sum(x.numel() * x.element_size() for w in own for x in w.values() if isinstance(x, torch.Tensor))


class SeqLMForCausalLM:
    PROFILE = "seq"   # the subset of native sources this family needs (livecc_b200.build.PROFILES)

    def __init__(self, config: SeqModelConfig, weights: SeqWeights, device: torch.device, max_tokens: int = 0):
        config.validate()
        if device.type != "cuda":
            raise _cabi.LiveCCNativeError("the hybrid sequence models need a CUDA (sm_100a) device; there is no CPU path")
        self.config, self.weights, self.device, self.dtype = config, weights, device, weights.dtype
        torch.cuda.set_device(device)
        self.ctx = _cabi.Context(device.index if device.index is not None else torch.cuda.current_device(), profile=self.PROFILE)
        self._native = self._build_native()
        attn = {i: (L.left.kv_heads, L.left.dim, L.left.vdim, L.left.chunk) for i, L in enumerate(config.layers) if L.type == "parallel"}
        # sliding-window attention: (kv heads, key size, value size, no chunks, window)
        attn.update({i: (L.attn.kv_heads, L.attn.dim, L.attn.vdim, 0, L.attn.window) for i, L in enumerate(config.layers) if L.type == "attention"})
        # a latent cache is one K pool of [latent | rotary key part] rows; a layer that reads another layer's cache has none
        attn.update({i: (1, L.latent.kv_rank + L.latent.rot_dim, 0, 0, L.latent.window) for i, L in enumerate(config.layers)
                     if L.type == "latent_attention" and L.latent.kv_from < 0})
        self._kv_source = {i: (L.latent.kv_from if L.latent.kv_from >= 0 else i) for i, L in enumerate(config.layers)
                           if L.type == "latent_attention"}
        pages = (max_tokens + PAGE_SIZE - 1) // PAGE_SIZE + 2 if max_tokens else 32
        self.pool = SeqStatePool(attn, self._native.state_floats(), self.dtype, device, initial_pages=pages)
        self._ensure_workspace(max(256, min(max_tokens, 4096)) if max_tokens else 1024, 64)
        self.generation_eos = config.eos_token_id
        self._logits_proc = torch.empty((config.vocab,), dtype=torch.float32, device=device)
        self._graphs = {}
        self.use_cuda_graph = os.environ.get("LIVECC_B200_NO_GRAPH", "0") != "1"
        self.last_stats = {}

    # -- construction --------------------------------------------------------------------------------------------
    @classmethod
    def from_state_dict(cls, config: SeqModelConfig, tensors, torch_dtype="bfloat16", device="cuda", max_tokens: int = 0):
        device = torch.device(device if ":" in str(device) else f"{device}:{torch.cuda.current_device()}")
        return cls(config, SeqWeights(config, tensors, _dtype_of(torch_dtype), device), device, max_tokens)

    @classmethod
    def from_pretrained(cls, model_path: str, torch_dtype="auto", device_map="cuda", max_tokens: int = 0, **_):
        """A directory with config.json and *.safetensors (bf16 tensors; names `embed`, `l<i>.norm1`, `l<i>.mix.*`,
        `l<i>.mlp.*`, `final.norm`, `head`; a Dynamic-Tanh norm adds `<norm>.b` and `<norm>.alpha`)."""
        from .checkpoint import iter_safetensors

        with open(os.path.join(model_path, "config.json")) as f:
            cfg = SeqModelConfig.from_json(json.load(f))
        return cls.from_state_dict(cfg, iter_safetensors(model_path), torch_dtype,
                                   device_map if isinstance(device_map, str) else "cuda", max_tokens)

    def _build_native(self) -> _cabi.SeqNativeModel:
        cfg, w = self.config, self.weights
        p = lambda x: x.data_ptr() if x is not None else None
        arr = (_cabi.SeqLayer * len(cfg.layers))()
        for i, (L, lw) in enumerate(zip(cfg.layers, w.layers)):
            e = arr[i]
            e.ff = L.ff
            e.norm1_f32 = p(lw["norm1"])
            e.norm1_bias_f32, e.norm1_alpha = p(lw.get("norm1_bias")), lw.get("norm1_alpha", 0.0)
            e.hc1_f32, e.hc2_f32 = p(lw.get("hc1")), p(lw.get("hc2"))
            e.a_kv_from = -1
            e.rot_inv_freq_f32, e.rot_mag = p(lw.get("rot_freq")), lw.get("rot_mag", 1.0)
            e.canon_w_f32 = p(lw.get("canon"))
            if L.type == "channel_delta":
                t = L.delta
                e.type = _cabi.MIX_DELTA
                e.d_heads, e.d_kv_heads, e.d_dim, e.d_vdim, e.d_conv, e.d_rank_a, e.d_rank_g = t.heads, t.kv_heads, t.dim, t.vdim, t.conv, t.rank_a, t.rank_g
                e.d_in, e.d_conv_w_f32, e.d_a_up, e.d_g_up, e.d_out = p(lw["d_in"]), p(lw["d_conv_w"]), p(lw["d_a_up"]), p(lw["d_g_up"]), p(lw["d_out"])
                e.d_dt_bias_f32, e.d_a_log_f32, e.d_norm_f32 = p(lw["d_dt_bias"]), p(lw["d_a_log"]), p(lw["d_norm"])
            elif L.type == "retention":
                t = L.retention
                e.type = _cabi.MIX_RETENTION
                e.t_heads, e.t_dim, e.t_vdim, e.t_rot_dims = t.heads, t.dim, t.vdim, t.rot.dims
                e.t_in, e.t_log_decay_f32, e.t_norm_f32, e.t_out = p(lw["t_in"]), p(lw["t_log_decay"]), p(lw["t_norm"]), p(lw["t_out"])
            elif L.type == "latent_attention":
                a = L.latent
                e.type = _cabi.MIX_LATENT
                e.a_heads, e.a_dim, e.a_rot_dim, e.a_vdim, e.a_rank, e.a_kv_from = a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank, a.kv_from
                e.a_scale = a.scale
                e.a_q_rank, e.a_window, e.a_gate = a.q_rank, a.window, int(a.gate)
                e.a_uq, e.a_q_norm_f32 = p(lw.get("a_uq")), p(lw.get("a_q_norm"))
                e.a_in, e.a_latent_norm_f32, e.a_uk_t, e.a_uv = p(lw["a_in"]), p(lw.get("a_latent_norm")), p(lw["a_uk_t"]), p(lw["a_uv"])
                e.a_sink_f32, e.a_out = p(lw.get("a_sink")), p(lw["a_out"])
            elif L.type == "attention":
                a = L.attn
                e.type = _cabi.MIX_ATTENTION
                e.m_heads, e.m_kv_heads, e.m_dim, e.m_vdim, e.m_window, e.m_chunk = a.heads, a.kv_heads, a.dim, a.vdim, a.window, 0
                e.m_rot_dims, e.m_rot_pairs, e.m_sink, e.m_value_keys = a.rot.dims, int(a.rot_pairs), int(a.sink), int(a.value_keys)
                e.m_gate = {"none": _cabi.GATE_NONE, "head": _cabi.GATE_HEAD, "channel": _cabi.GATE_CHANNEL}[a.gate]
                e.m_scale = a.scale
                e.m_unit_norm, e.m_vmix_role, e.m_vmix, e.m_temp_f32 = int(a.unit_norm), lw.get("m_vmix_role", 0), lw.get("m_vmix", 0.0), p(lw.get("m_temp"))
                e.m_in, e.m_qnorm_f32, e.m_knorm_f32, e.m_out = p(lw["m_in"]), p(lw.get("m_qnorm")), p(lw.get("m_knorm")), p(lw["m_out"])
            elif L.type == "mamba2":
                s = L.ssd
                e.type = _cabi.MIX_SSD
                e.s_heads, e.s_vdim, e.s_state, e.s_groups, e.s_conv, e.s_norm_groups = s.heads, s.vdim, s.state, s.groups, s.conv, s.norm_groups
                e.s_in, e.s_conv_w_f32, e.s_conv_b_f32 = p(lw["s_in"]), p(lw["s_conv_w"]), p(lw["s_conv_b"])
                e.s_dt_bias_f32, e.s_a_log_f32, e.s_skip_f32 = p(lw["s_dt_bias"]), p(lw["s_a_log"]), p(lw["s_skip"])
                e.s_norm_f32, e.s_out = p(lw["s_norm"]), p(lw["s_out"])
            else:
                l, r = L.left, L.right
                e.type = _cabi.MIX_PARALLEL
                e.l_heads, e.l_kv_heads, e.l_dim, e.l_vdim, e.l_chunk, e.l_scale = l.heads, l.kv_heads, l.dim, l.vdim, l.chunk, l.scale
                e.r_heads, e.r_dim, e.r_vdim, e.r_rank, e.r_tau = r.heads, r.dim, r.vdim, r.rank, r.tau
                e.l_in, e.l_in_bias_f32, e.l_qnorm_f32, e.l_knorm_f32 = p(lw["l_in"]), p(lw["l_in_bias"]), p(lw["l_qnorm"]), p(lw["l_knorm"])
                e.l_in_bias = p(lw["l_in_bias_st"])
                e.l_out, e.l_branch_norm_f32 = p(lw["l_out"]), p(lw["l_branch_norm"])
                e.r_in, e.r_decay_up, e.r_decay_bias_f32 = p(lw["r_in"]), p(lw["r_decay_up"]), p(lw["r_decay_bias"])
                e.r_norm_f32, e.r_out, e.r_branch_norm_f32 = p(lw["r_norm"]), p(lw["r_out"]), p(lw["r_branch_norm"])
            if L.moe:
                x = L.moe
                e.ff_kind = _cabi.FF_MOE
                e.e_experts, e.e_top, e.e_ff, e.e_shared_ff, e.e_scale = x.experts, x.top, x.ff, x.shared_ff, x.scale
                e.e_router_kind = {"softmax": _cabi.ROUTER_SOFTMAX, "topk_softmax": _cabi.ROUTER_TOPK_SOFTMAX}.get(x.router, _cabi.ROUTER_SIGMOID)
                e.e_identity, e.e_groups, e.e_keep, e.e_limit = x.identity, x.groups, x.keep, x.limit
                e.e_act = {"clamp_glu": _cabi.EXPERT_CLAMP_GLU, "silu_glu": _cabi.EXPERT_SILU_GLU}.get(x.act, _cabi.EXPERT_RELU2)
                e.e_up_il16 = lw.get("e_up_il16", 0)
                e.norm2_f32, e.e_router, e.e_correction_f32 = p(lw.get("norm2")), p(lw["e_router"]), p(lw.get("e_correction"))
                e.e_up, e.e_down = p(lw["e_up"]), p(lw["e_down"])
                e.e_shared_up, e.e_shared_down = p(lw.get("e_shared_up")), p(lw.get("e_shared_down"))
            elif L.ff:
                e.ff_kind = _cabi.FF_MLP if cfg.dense == "mlp" else _cabi.FF_GLU
                e.norm2_f32, e.ff_in, e.ff_out = p(lw.get("norm2")), p(lw["ff_in"]), p(lw["ff_out"])
        desc = _cabi.SeqModelDesc(
            width=cfg.width, vocab=cfg.vocab, n_layers=len(cfg.layers),
            dtype=_cabi.DT_F32 if self.dtype == torch.float32 else _cabi.DT_BF16, rows_padded8=1, eps=cfg.eps, alpha=cfg.alpha,
            embed_scale=cfg.embed_scale, logit_softcap=cfg.logit_softcap,
            block={"prenorm_hc": _cabi.BLOCK_PRENORM_HC, "parallel": _cabi.BLOCK_PARALLEL, "branchnorm": _cabi.BLOCK_BRANCHNORM}.get(cfg.block, _cabi.BLOCK_POSTNORM),
            streams=cfg.streams, canon_taps=cfg.canon_taps,
            norm_kind=_cabi.NORM_DYT if cfg.norm == "dyt" else _cabi.NORM_RMS, final_norm_alpha=w.final_norm_alpha,
            logit_scale=cfg.logit_scale, final_norm_bias_f32=p(w.final_norm_bias),
            embed=p(w.embed), inv_freq_f32=p(w.inv_freq),
            final_norm_f32=p(w.final_norm), head=p(w.head), layers=arr)
        return _cabi.SeqNativeModel(self.ctx, desc, keepalive=(arr, w))

    def _ensure_workspace(self, tokens: int, want: int):
        n = self._native
        if tokens <= n.cap_tokens and want <= n.cap_want:
            return
        torch.cuda.synchronize(self.device)
        n.bind_workspace(max(tokens, n.cap_tokens), max(want, n.cap_want), self.device)
        self._graphs = {}

    # -- HF-surface helpers ----------------------------------------------------------------------------------------
    def eval(self):
        return self

    def to(self, *_, **__):
        return self

    def new_cache(self) -> SeqCache:
        return SeqCache(self.pool)

    def kernel_launches(self) -> int:
        return _cabi.launch_count()

    # -- one step ----------------------------------------------------------------------------------------------------
    def _entry(self, cache: SeqCache, ids_dev: torch.Tensor, n_new: int, keep: list, device_pos: bool) -> _cabi.SeqEntry:
        nl = len(self.config.layers)
        pool = self.pool
        st = (C.c_void_p * nl)(*[(pool.state[i][cache.slot].data_ptr() if pool.state[i] is not None else None) for i in range(nl)])
        src = self._kv_source                       # latent-attention layers: whose K pool they read
        kp = (C.c_void_p * nl)(*[(pool.k[src.get(i, i)].data_ptr() if src.get(i, i) in pool.k else None) for i in range(nl)])
        vp = (C.c_void_p * nl)(*[(pool.v[i].data_ptr() if pool.v.get(i) is not None else None) for i in range(nl)])
        keep += [st, kp, vp]
        return _cabi.SeqEntry(n_new=n_new, past=cache.seq_len, ids=ids_dev.data_ptr(), page_table=cache.page_table.data_ptr(),
                              scalars=cache.scalars.data_ptr() if device_pos else None, layer_state=st, k_pages=kp, v_pages=vp)

    @torch.inference_mode()
    def forward_step(self, entries: Sequence[Tuple[SeqCache, Sequence[int]]], want: Optional[Sequence[Sequence[int]]] = None,
                     layer_dump: bool = False):
        """One step of the scheduler: each entry brings a sequence's next tokens (a prompt portion of any length, or one
        token); `want[e]` lists the places among entry e's tokens whose logits are asked for. Linear layers and row ops run
        over the rows of all entries at once, the sequence mixers per entry from the state earlier steps left. Returns
        fp32 logits [sum(len(want[e])), vocab] in entry order (and, with layer_dump, the residual stream after every layer
        [layers, rows, width])."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        if len({id(c) for c, _ in entries}) != len(entries):
            raise ValueError("the same sequence appears twice in one step")
        want = want if want is not None else [[] for _ in entries]
        rows, want_rows, ents, keep = 0, [], [], []
        all_ids = []
        for (cache, ids), w in zip(entries, want):
            if cache.pool is not self.pool or cache.slot is None:
                raise TypeError("the cache does not belong to this model (or was released)")
            ids = [int(x) for x in (ids.tolist() if isinstance(ids, torch.Tensor) else ids)]
            if not ids:
                raise ValueError("an entry without tokens")
            if any(not 0 <= k < len(ids) for k in w):
                raise ValueError("a wanted place outside the entry's tokens")
            want_rows += [rows + int(k) for k in w]
            all_ids += ids
            rows += len(ids)
        self._ensure_workspace(rows, max(len(want_rows), 1))
        ids_dev = torch.tensor(all_ids, dtype=torch.int64).to(self.device)
        r0 = 0
        for (cache, ids), _w in zip(entries, want):
            n = len(ids)
            cache.ensure_tokens(cache.seq_len + n)   # may move the pool: entries are built after all allocations
            r0 += n
        r0 = 0
        for (cache, ids), _w in zip(entries, want):
            n = len(ids)
            ents.append(self._entry(cache, ids_dev[r0:r0 + n], n, keep, device_pos=False))
            r0 += n
        nw = len(want_rows)
        want_dev = torch.tensor(want_rows, dtype=torch.int32).to(self.device) if nw else None
        logits = torch.empty((nw, self.config.vocab), dtype=torch.float32, device=self.device) if nw else None
        dump = torch.empty((len(self.config.layers), rows, self.config.width), dtype=torch.float32, device=self.device) if layer_dump else None
        self._native.forward(ents, PAGE_SIZE, want_dev, nw, logits, None, dump)
        for (cache, ids), _w in zip(entries, want):
            cache.advance(len(ids))
        return (logits, dump) if layer_dump else logits

    # -- generation ----------------------------------------------------------------------------------------------------
    def _sampling(self, repetition_penalty, max_new_tokens, eos_token_id) -> _cabi.Sampling:
        eos = self.generation_eos if eos_token_id is None else eos_token_id
        eos = [int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos])]
        return _cabi.Sampling(float(repetition_penalty), -1, 0.0, 0.0, eos[0], int(max_new_tokens),
                              1.0 / float(repetition_penalty), eos[1] if len(eos) > 1 else -1)

    @torch.inference_mode()
    def generate(self, input_ids: torch.Tensor, past_key_values: Optional[SeqCache] = None, max_new_tokens: int = 16,
                 repetition_penalty: float = 1.0, eos_token_id=None, do_sample: Optional[bool] = None,
                 return_dict_in_generate: bool = True, output_logits: bool = False, prefill_chunk: int = 0, **unsupported):
        """Greedy generation. input_ids: [1, L] = the full id history; the cache decides how many trailing ids are new.
        The prompt runs as one step (or in portions of `prefill_chunk` tokens), then every token is one decode step
        followed by the library's token-selection kernel; positions, ids and the stop flag live on the device, the decode
        step is captured once as a CUDA graph and replayed, and the host synchronises once per call."""
        if unsupported:
            raise TypeError(f"generate() got unsupported arguments {sorted(unsupported)}")
        if do_sample:
            raise NotImplementedError("the native token selection is greedy")
        if input_ids is None or input_ids.dim() != 2 or input_ids.shape[0] != 1:
            raise ValueError("input_ids must be [1, L] (one sequence per call)")
        if max_new_tokens < 1:
            raise ValueError("max_new_tokens must be >= 1")
        cache = past_key_values if past_key_values is not None else self.new_cache()
        ids = input_ids[0].tolist()
        L, past = len(ids), cache.seq_len
        if L <= past:
            raise ValueError(f"input_ids has {L} ids but the cache already holds {past}")
        sp = self._sampling(repetition_penalty, max_new_tokens, eos_token_id)
        V = self.config.vocab
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record()
        # ---- prompt ----
        new = ids[past:]
        step = prefill_chunk if prefill_chunk > 0 else len(new)
        for a in range(0, len(new) - step, step) if step < len(new) else []:
            self.forward_step([(cache, new[a:a + step])])
        done = (len(new) - 1) // step * step if step < len(new) else 0
        last = new[done:]
        logits = self.forward_step([(cache, last)], [[len(last) - 1]])
        # ---- first token + decode steps ----
        cache.ensure_seq_capacity(L + max_new_tokens + 1)
        cache.ensure_tokens(L + max_new_tokens)
        cache.seq_buf[:L].copy_(torch.tensor(ids, dtype=torch.int64))
        cache.scalars.copy_(torch.tensor([L, L, 0, 0, L, 0, 0, 0], dtype=torch.int32))
        raw = torch.empty((1, V), dtype=torch.float32, device=self.device)
        raw.copy_(logits)
        logits_out = [raw[0].clone()] if output_logits else None
        self._select(raw, cache, sp, advance=0)
        n_steps = max_new_tokens - 1
        hist = torch.empty((n_steps, V), dtype=torch.float32, device=self.device) if output_logits and n_steps else None
        ev[1].record()
        if n_steps:
            self._run_decode(cache, raw, sp, n_steps, hist)
        ev[2].record()
        sc = cache.scalars.tolist()                      # the one host sync of the decode phase
        n_gen = sc[_cabi.SC_N_GENERATED]
        # the device advanced the position; pages behind the last chunk go back as in a teacher-forced step
        cache.seq_len = L
        cache.advance(sc[_cabi.SC_KV_LEN] - L)
        seq = cache.seq_buf[: L + n_gen].clone().view(1, -1)
        if output_logits and hist is not None:
            logits_out += list(hist[: max(n_gen - 1, 0)])
        self.last_stats = {"prefill_tokens": len(new), "generated": n_gen, "kv_len": cache.seq_len,
                           "prefill_ms": ev[0].elapsed_time(ev[1]), "decode_ms": ev[1].elapsed_time(ev[2])}
        out = GenerateOutput(sequences=seq, past_key_values=cache, logits=logits_out[:n_gen] if output_logits else None)
        return out if return_dict_in_generate else out.sequences

    def _select(self, raw: torch.Tensor, cache: SeqCache, sp: _cabi.Sampling, advance: int):
        self._logits_proc.copy_(raw[0])
        self.ctx.call("lcc_sample_greedy", _cabi._ptr(raw), _cabi._ptr(self._logits_proc), _cabi._i(self.config.vocab),
                      _cabi._ptr(cache.seq_buf), _cabi._ptr(cache.scalars), C.byref(sp), _cabi._i(advance), None, None,
                      _cabi._i(self.config.width), _cabi.Context.stream_ptr())

    def _decode_once(self, cache: SeqCache, raw: torch.Tensor, sp: _cabi.Sampling, keep: list):
        """One token, all bookkeeping on the device: the step reads the last id (seq[SEQ_LEN - 1]) and the number of cached
        tokens (KV_LEN) from the sequence's scalars; the selection kernel appends the next id and advances both."""
        ent = self._entry(cache, cache.seq_buf, 1, keep, device_pos=True)
        self._native.forward([ent], PAGE_SIZE, self._want0, 1, raw, None, None)
        self._select(raw, cache, sp, advance=1)

    def _run_decode(self, cache: SeqCache, raw: torch.Tensor, sp: _cabi.Sampling, n_steps: int, hist):
        if not hasattr(self, "_want0"):
            self._want0 = torch.zeros(1, dtype=torch.int32, device=self.device)
        if not self.use_cuda_graph:
            keep: list = []
            for i in range(n_steps):
                self._decode_once(cache, raw, sp, keep)
                if hist is not None:
                    hist[i].copy_(raw[0])
            return
        key = (self.pool.generation, cache.table_generation, cache.scalars.data_ptr(), cache.seq_buf.data_ptr(),
               cache.page_table.data_ptr(), cache.slot, self._native.workspace.data_ptr(),
               sp.repetition_penalty, sp.eos_token_id, sp.eos_token_id2, sp.max_new_tokens)
        ent = self._graphs.get(key)
        first = 0
        if ent is None:
            if len(self._graphs) > 16:
                self._graphs.clear()
            gkeep: list = []
            graw = torch.empty_like(raw)
            self._decode_once(cache, graw, sp, gkeep)   # eager once: lazy module loading, kernel attributes
            if hist is not None:
                hist[0].copy_(graw[0])
            first = 1
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side, capture_error_mode="thread_local"):
                    self._decode_once(cache, graw, sp, gkeep)
            torch.cuda.current_stream(self.device).wait_stream(side)
            ent = self._graphs[key] = (g, gkeep, graw)
        g, _, graw = ent
        for i in range(first, n_steps):
            g.replay()
            if hist is not None:
                hist[i].copy_(graw[0])
