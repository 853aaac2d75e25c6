"""Prefill and decode throughput of the hybrid sequence models at layer sizes that resemble a real model's, beside the
framework's Qwen2-style decoder (the closest existing model) at equal width, depth and feed-forward size. Random weights.
Used by `bench.py --arch seq`; every number is timed with CUDA events on the launching stream after warm-up, and the
weights of every size are larger than L2, so each step streams them from HBM."""
from __future__ import annotations

import json
from typing import Dict, List

import torch

from .checkpoint import synthetic_seq_tensors
from .config import LiveCCConfig, SeqModelConfig, TextConfig, VisionConfig

# name -> (width, layers, feed-forward, attention chunk)
SIZES = {
    "w2048": (2048, 8, 5632, 1024),
    "w4096": (4096, 4, 11008, 1024),
}
PATTERN = ("mamba2", "mamba2", "mamba2", "parallel")


def seq_config(width: int, n_layers: int, ff: int, chunk: int, vocab: int = 32768) -> SeqModelConfig:
    """State-space layers with 2x expansion (64-channel heads, 128 states), every fourth layer a parallel layer with
    128-wide attention heads (8 query heads per key/value head) beside gated linear attention, feed-forward on the
    parallel layers."""
    layers = []
    for i in range(n_layers):
        if PATTERN[i % len(PATTERN)] == "mamba2":
            layers.append({"type": "mamba2", "mlp": None,
                           "mixer": dict(heads=2 * width // 64, vdim=64, state=128, groups=8, conv=4, norm_groups=8)})
        else:
            heads = width // 128
            layers.append({"type": "parallel", "mlp": {"ff": ff, "kind": "dense"},
                           "mixer": {"left": dict(heads=heads, kv_heads=max(1, heads // 8), dim=128, vdim=128, mask={"size": chunk},
                                                  scale=128 ** -0.5),
                                     "right": dict(heads=width // 256, dim=128, vdim=256, tau=8.0)}})
    return SeqModelConfig.from_json({"architecture": "Bimopel", "vocab": vocab, "width": width, "layers": layers,
                                     "norm": {"eps": 1e-5}, "postln_alpha": 2.0, "embedding": {"scale": width ** 0.5},
                                     "logit_softcap": 50.0})


def kedelorn_config(width: int, n_layers: int, ff: int, vocab: int = 32768) -> SeqModelConfig:
    """Two residual streams; layers in the pattern latent attention, latent attention reading the first one's cache,
    retention, retention. Latent attention: 128 + 64 channel query heads, 192 latent + 64 rotary cache channels per token,
    128-channel values. Retention: 128-channel keys, 256-channel values, decays 1 - 2^-(5+h). Every layer has 16 experts
    of width ff/4 (2 per token) and a shared expert of width ff/2: the active feed-forward width per token equals the dense
    `ff` of the models beside it."""
    heads, layers = width // 128, []
    rot = {"dims": 64, "base": 10000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    mlp = {"kind": "moe", "expert": {"ff": ff // 4 // 8 * 8}, "router": {"experts": 16, "top": 2, "scale": 2.5},
           "shared": {"ff": ff // 2 // 8 * 8}}
    for i in range(n_layers):
        k = i % 4
        if k < 2:
            mx = dict(heads=heads, dim=128, rot_dim=64, vdim=128, kv_rank=192, scale=192 ** -0.5, rot=rot)
            if k == 1:
                mx["kv_from"] = i - 1
            layers.append({"type": "latent_attention", "mixer": mx, "mlp": mlp})
        else:
            rh = width // 256
            layers.append({"type": "retention", "mlp": mlp,
                           "mixer": dict(heads=rh, dim=128, vdim=256, decay=[1.0 - 2.0 ** (-5 - (h % 8)) for h in range(rh)],
                                         rot={"dims": 128, "base": 10000.0})})
    return SeqModelConfig.from_json({"architecture": "Kedelorn", "vocab": vocab, "width": width, "streams": 2, "layers": layers,
                                     "norm": {"eps": 1e-6}})


def dibedra_config(width: int, n_layers: int, ff: int, window: int, vocab: int = 32768) -> SeqModelConfig:
    """Parallel blocks; every layer sliding-window attention with 128-channel heads (8 query heads per key/value head, the
    first 64 channels rotated, long-context frequencies). The first layer has a two-matrix feed-forward of width 3 ff / 2,
    every other layer 16 experts of width ff/4 and 2 identity experts, 4 per token out of the best 6 of 9 groups: a token
    whose four choices are real experts reads 3 x width x ff feed-forward weights, the dense gated `ff` of the models beside it."""
    heads, layers = width // 128, []
    rot = {"dims": 64, "base": 250000.0, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    mx = dict(heads=heads, kv_heads=max(1, heads // 8), dim=128, vdim=128, mask={"size": window}, rot=rot, scale=128 ** -0.5)
    moe = {"kind": "moe", "expert": {"ff": ff // 4 // 8 * 8, "limit": 7.0},
           "router": {"experts": 16, "identity": 2, "top": 4, "groups": {"count": 9, "keep": 6}}}
    for i in range(n_layers):
        layers.append({"type": "attention", "mixer": mx, "mlp": {"kind": "dense", "ff": 3 * ff // 2 // 8 * 8} if i == 0 else moe})
    return SeqModelConfig.from_json({"architecture": "Dibedra", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-6},
                                     "logit_scale": 0.5})


def lugizen_config(width: int, n_layers: int, ff: int, window: int, vocab: int = 32768) -> SeqModelConfig:
    """Sublayers normed on their output behind a 4-tap convolution over time; layers in the pattern delta rule, delta rule,
    attention, latent attention. Delta rule: width/128 heads of 128 key and 128 value channels, 4-tap q/k/v convolutions,
    decay and gate bottlenecks of 64 channels. Attention: 128-channel heads, 8 query heads per key/value head, the first 64
    channels rotated, values mixed across the attention layers. Latent attention: 128 + 64 channel query heads through a query
    latent of 3/8 width, 192 latent + 64 rotary cache channels per token, 128-channel values, a window of `window` positions.
    The first layer has a two-matrix feed-forward of width 3 ff / 2, every other layer 16 gated experts of width ff/4, 4 per
    token: every token reads 3 x width x ff feed-forward weights, the dense gated `ff` of the models beside it."""
    heads, layers = width // 128, []
    moe = {"kind": "moe", "expert": {"ff": ff // 4 // 16 * 16}, "router": {"experts": 16, "top": 4}}
    for i in range(n_layers):
        k = i % 4
        if k < 2:
            L = {"type": "channel_delta", "mixer": dict(heads=heads, kv_heads=heads, dim=128, vdim=128, conv=4, decay_rank=64, gate_rank=64)}
        elif k == 2:
            L = {"type": "attention", "mixer": dict(heads=heads, kv_heads=max(1, heads // 8), dim=128, vdim=128, rot={"dims": 64, "base": 10000.0},
                                                    scale=128 ** -0.5, v_mix=True)}
        else:
            L = {"type": "latent_attention", "mixer": dict(heads=heads, dim=128, rot_dim=64, vdim=128, kv_rank=192, q_rank=3 * width // 8,
                                                           mask={"size": window}, rot={"dims": 64, "base": 10000.0}, scale=192 ** -0.5)}
        L["mlp"] = {"kind": "dense", "ff": 3 * ff // 2 // 8 * 8} if i == 0 else moe
        layers.append(L)
    return SeqModelConfig.from_json({"architecture": "Lugizen", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-6},
                                     "canon": {"taps": 4}})


def qwen_config(width: int, n_layers: int, ff: int, vocab: int = 32768) -> LiveCCConfig:
    heads = width // 128
    return LiveCCConfig(
        text_config=TextConfig(hidden_size=width, intermediate_size=ff, num_hidden_layers=n_layers, num_attention_heads=heads,
                               num_key_value_heads=max(1, heads // 8)),
        vision_config=VisionConfig(depth=1, embed_dim=320, hidden_size=width, num_heads=4),
        name=f"qwen2-w{width}-l{n_layers}").with_vocab(vocab)


def _ids(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab - 64, (1, n), generator=g)


def _median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def time_seq(model, prompt_len: int, new_tokens: int, steps: int, warmup: int) -> Dict:
    pre, dec = [], []
    for i in range(warmup + steps):
        out = model.generate(_ids(prompt_len, model.config.vocab, i), max_new_tokens=new_tokens + 1, eos_token_id=-1)
        out.past_key_values.release()
        if i >= warmup:
            pre.append(model.last_stats["prefill_ms"])
            dec.append(model.last_stats["decode_ms"] / max(model.last_stats["generated"] - 1, 1))
    return {"prefill_ms": _median(pre), "prefill_tok_s": prompt_len / _median(pre) * 1e3, "decode_ms_per_token": _median(dec),
            "decode_tok_s": 1e3 / _median(dec)}


def time_qwen(model, prompt_len: int, new_tokens: int, steps: int, warmup: int) -> Dict:
    pre, dec = [], []
    saved = model.generation_config.eos_token_id
    model.generation_config.eos_token_id = -1            # random weights: never stop early
    for i in range(warmup + steps):
        out = model.generate(input_ids=_ids(prompt_len, model.config.text_config.vocab_size, i), max_new_tokens=new_tokens + 1)
        out.past_key_values.release()
        if i >= warmup:
            st = model.last_stats
            pre.append(st["prefill_ms"])
            dec.append(st["decode_ms"] / max(st["generated"] - 1, 1))
    model.generation_config.eos_token_id = saved
    return {"prefill_ms": _median(pre), "prefill_tok_s": prompt_len / _median(pre) * 1e3, "decode_ms_per_token": _median(dec),
            "decode_tok_s": 1e3 / _median(dec)}


def active_weight_bytes(model) -> int:
    """Bytes of weights one decode step reads: everything but the embedding table (one row is read) and, in a routed
    feed-forward, the experts that were not chosen."""
    n = model.weights.nbytes() - model.weights.embed.numel() * model.weights.embed.element_size()
    for L, w in zip(model.config.layers, model.weights.layers):
        if L.moe:
            per = (w["e_up"].numel() + w["e_down"].numel()) * w["e_up"].element_size() // L.moe.experts
            n -= per * (L.moe.experts - L.moe.top)
    return n


def run(sizes: List[str], prompt_lens: List[int], new_tokens: int, steps: int, warmup: int, dtype: str = "bfloat16",
        design: str = "Bimopel") -> Dict:
    from .engine import LiveCCB200ForConditionalGeneration
    from .seq_engine import SeqLMForCausalLM

    out = {}
    for name in sizes:
        width, n_layers, ff, chunk = SIZES[name]
        rec = {}
        arms = {"Bimopel": ["bimopel"], "Kedelorn": ["kedelorn", "bimopel"], "Dibedra": ["dibedra", "kedelorn"],
                "Lugizen": ["lugizen", "kedelorn"]}[design]
        make = {"bimopel": lambda: seq_config(width, n_layers, ff, chunk), "kedelorn": lambda: kedelorn_config(width, n_layers, ff),
                "dibedra": lambda: dibedra_config(width, n_layers, ff, chunk), "lugizen": lambda: lugizen_config(width, n_layers, ff, chunk)}
        for label, cfg in [(a, make[a]()) for a in arms]:
            m = SeqLMForCausalLM.from_state_dict(cfg, synthetic_seq_tensors(cfg, seed=7, device="cuda"), dtype,
                                                 max_tokens=max(prompt_lens) + new_tokens + 64)
            rec["weights_gb" if label == "bimopel" else label + "_weights_gb"] = round(m.weights.nbytes() / 1e9, 3)
            rec[label + "_decode_read_gb"] = round(active_weight_bytes(m) / 1e9, 3)
            rec[label] = {}
            for S in prompt_lens:
                rec[label][f"S{S}"] = time_seq(m, S, new_tokens, steps, warmup)
            del m
            torch.cuda.empty_cache()
        rec["qwen2"] = {}
        q = LiveCCB200ForConditionalGeneration.from_synthetic(qwen_config(width, n_layers, ff))
        rec["qwen2_weights_gb"] = round(q.weights.nbytes() / 1e9, 3)
        for S in prompt_lens:
            rec["qwen2"][f"S{S}"] = time_qwen(q, S, new_tokens, steps, warmup)
        del q
        torch.cuda.empty_cache()
        out[name] = rec
    return out


def main(args, design: str = "Bimopel") -> Dict:
    """bench.py --arch seq | kedelorn | dibedra | lugizen: one JSON line; `value` = decode tokens/s of the first size at the first prompt length."""
    sizes = [s for s in (args.seq_sizes.split(",") if args.seq_sizes else list(SIZES)) if s in SIZES]
    lens = [int(x) for x in args.seq_prompt.split(",")]
    res = run(sizes, lens, args.max_new_tokens if args.max_new_tokens > 16 else 64, args.steps, max(args.warmup, 3), design=design)
    first = res[sizes[0]][design.lower()][f"S{lens[0]}"]
    return {"metric": "decode_tokens_per_s", "value": first["decode_tok_s"], "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": first["decode_ms_per_token"], "higher_is_better": True, "dtype": "bf16",
            "data": "synthetic (random weights, random ids)", "vs_baseline": None,
            "config": {"model": f"{design} {sizes[0]} beside " + {"Kedelorn": "Bimopel and the ", "Dibedra": "Kedelorn and the ", "Lugizen": "Kedelorn and the "}.get(design, "") +
                                "Qwen2-style decoder of equal width/depth/ff", "global_batch": 1,
                       "seq_len": lens[0], "parallelism": "1 gpu", "l2": "weights of every size exceed L2"},
            "sizes": res}
