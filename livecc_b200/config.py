"""Model hyper-parameters of the LiveCC hot path (Qwen2-VL architecture).

Field names follow transformers' Qwen2VLConfig / Qwen2VLTextConfig / Qwen2VLVisionConfig
(SP/transformers/models/qwen2_vl/configuration_qwen2_vl.py:31-41,100-101,159-163) so that the
reference-facing code reads `model.config.eos_token_id`, `.video_token_id` exactly as
REF/demo/infer.py:171 and REF/livecc-utils/src/livecc_utils/generation_patch.py:37 do.
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class VisionConfig:
    depth: int = 32
    embed_dim: int = 1280
    hidden_size: int = 3584  # merger output = text hidden size
    mlp_ratio: int = 4
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 14
    spatial_merge_size: int = 2
    temporal_patch_size: int = 2

    @property
    def head_dim(self) -> int:
        return self.embed_dim // self.num_heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size

    @property
    def mlp_dim(self) -> int:
        return self.embed_dim * self.mlp_ratio


@dataclass
class TextConfig:
    vocab_size: int = 152064
    hidden_size: int = 3584
    intermediate_size: int = 18944
    num_hidden_layers: int = 28
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    mrope_section: tuple = (16, 24, 24)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


@dataclass
class LiveCCConfig:
    text_config: TextConfig = field(default_factory=TextConfig)
    vision_config: VisionConfig = field(default_factory=VisionConfig)
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652
    vision_end_token_id: int = 151653
    bos_token_id: int = 151643
    eos_token_id: int = 151645
    pad_token_id: int = 151643
    im_start_token_id: int = 151644
    newline_token_id: int = 198
    name: str = "livecc-7b"

    def special_token_ids(self) -> dict:
        """Token string -> id for the special tokens the chat template emits."""
        return {
            "<|endoftext|>": self.bos_token_id,
            "<|im_start|>": self.im_start_token_id,
            "<|im_end|>": self.eos_token_id,
            "<|vision_start|>": self.vision_start_token_id,
            "<|vision_end|>": self.vision_end_token_id,
            "<|image_pad|>": self.image_token_id,
            "<|video_pad|>": self.video_token_id,
        }

    # -- factories --------------------------------------------------------------------------
    @staticmethod
    def livecc_7b() -> "LiveCCConfig":
        """LiveCC-7B = Qwen2-VL-7B dims (SURVEY.md §8 header)."""
        return LiveCCConfig()

    @staticmethod
    def small(layers: int = 2, vit_depth: int = 2) -> "LiveCCConfig":
        """Parity-test config: the 7B head geometry (decoder head_dim 128 with GQA 7:1, ViT
        head_dim 80) at a fraction of the width/depth, so that the CPU oracle finishes in seconds."""
        return LiveCCConfig(
            text_config=TextConfig(hidden_size=1792, intermediate_size=4864, num_hidden_layers=layers,
                                   num_attention_heads=14, num_key_value_heads=2),
            vision_config=VisionConfig(depth=vit_depth, embed_dim=320, hidden_size=1792, num_heads=4),
            name=f"livecc-small-l{layers}v{vit_depth}",
        ).with_vocab(16384)

    def with_vocab(self, vocab_size: int) -> "LiveCCConfig":
        """Shrinks the vocabulary (CPU-oracle speed) and relocates the special ids to its top."""
        self.text_config.vocab_size = vocab_size
        top = vocab_size - 32
        self.bos_token_id = self.pad_token_id = top + 0
        self.im_start_token_id = top + 1
        self.eos_token_id = top + 2
        self.vision_start_token_id = top + 9
        self.vision_end_token_id = top + 10
        self.image_token_id = top + 12
        self.video_token_id = top + 13
        return self

    def validate(self) -> None:
        t, v = self.text_config, self.vision_config
        if t.head_dim != 128:
            raise ValueError("decoder kernels are specialised for head_dim 128")
        if v.head_dim != 80:
            raise ValueError("ViT attention kernel is specialised for head_dim 80")
        if sum(t.mrope_section) * 2 != t.head_dim:
            raise ValueError("mrope_section must sum to head_dim/2")
        if v.hidden_size != t.hidden_size:
            raise ValueError("merger output must equal text hidden size")
        if t.intermediate_size % 32 or t.hidden_size % 8 or v.embed_dim % 8:
            raise ValueError("unsupported dims")


# ------------------------------------------------------------------------------------------------
# Hybrid sequence models (decoder-only language models built from recurrent and local-attention mixers)
# ------------------------------------------------------------------------------------------------
@dataclass
class SsdMixerConfig:
    """Scalar-decay state-space mixer: heads x vdim value channels, `state` key channels shared by heads/groups heads."""
    heads: int
    vdim: int
    state: int
    groups: int = 1
    conv: int = 4
    norm_groups: int = 1

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state

    @property
    def proj_rows(self) -> int:
        return self.inner + self.conv_channels + self.heads


@dataclass
class ChunkAttnConfig:
    """Attention inside chunks of `chunk` positions (0 = plain causal) with a softmax sink and a per-head output gate."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    chunk: int
    scale: float


@dataclass
class GlaConfig:
    """Gated linear attention with per-key-channel decays sigmoid(z)^(1/tau); z comes through a rank-`rank` bottleneck."""
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int = 0   # read from the tensor shapes when 0


@dataclass
class RotaryConfig:
    """Rotate-half rotary positions on the first `dims` channels of a head: pair i turns by p * base^(-2i/dims). `scaling`
    (factor, original, fast, slow) interpolates the slow pairs for contexts beyond `original` positions (YaRN: pairs that
    turn fewer than `slow` times over the original context are divided by `factor`, pairs that turn more than `fast` times
    are kept, a linear ramp in between) and multiplies cos and sin by 0.1 ln(factor) + 1."""
    dims: int
    base: float
    scaling: dict = None

    @staticmethod
    def from_json(d: dict, dims: int = 0) -> "RotaryConfig":
        """`dims` is the default when the dictionary names none (the rotated part of a latent-attention head)."""
        sc = d.get("scaling")
        return RotaryConfig(dims=int(d.get("dims", dims)), base=float(d["base"]),
                            scaling={k: float(sc[k]) for k in ("factor", "original", "fast", "slow")} if sc else None)

    def to_json(self) -> dict:
        out = dict(dims=self.dims, base=self.base)
        if self.scaling:
            out["scaling"] = dict(self.scaling)
        return out

    def frequencies(self):
        """([dims/2] frequencies in float64, factor on cos and sin)."""
        import math

        half = self.dims // 2
        f = [self.base ** (-2.0 * i / self.dims) for i in range(half)]
        if not self.scaling:
            return f, 1.0
        sc = self.scaling
        log_base = math.log(self.base)

        def pair_index(turns):   # the (fractional) pair that makes `turns` full turns over the original context
            return self.dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * log_base)

        lo = max(math.floor(pair_index(sc["fast"])), 0)
        hi = min(math.ceil(pair_index(sc["slow"])), self.dims - 1)
        out = []
        for i in range(half):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            out.append(f[i] / sc["factor"] * ramp + f[i] * (1.0 - ramp))
        return out, 0.1 * math.log(sc["factor"]) + 1.0


@dataclass
class RetentionConfig:
    """Linear attention with one fixed decay per head and no normaliser: S <- decay_h S + k v^T, o = S^T q; rotary q and k,
    k scaled by dim^-1/2; each head's output brought to unit rms, times silu(gate)."""
    heads: int
    dim: int
    vdim: int
    decay: list
    rot: RotaryConfig


@dataclass
class LatentAttnConfig:
    """Causal softmax attention whose keys and values are per-head up-projections of a cached latent of `kv_rank` channels,
    plus `rot_dim` rotary channels shared by all heads; a per-head sink logit in the denominator and a per-head sigmoid
    gate. `kv_from` >= 0: the layer has no latent projection and reads that layer's cache."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig
    kv_from: int = -1
    q_rank: int = 0       # > 0: the queries come through a latent of that many channels (RMS norm with a weight, then an up-projection)
    window: int = 0       # > 0: row i sees j with 0 <= i - j < window
    gate: bool = True     # the per-head sigmoid gate
    sink: bool = True     # the per-head sink logit (False: ordinary softmax)


@dataclass
class MoeConfig:
    """Routed feed-forward: `experts` experts of width `ff`, `top` per token chosen by score + correction, weighted by
    score * scale (never renormalised); a shared expert of width `shared_ff` (0: none) behind a scalar sigmoid gate.
    `router`: "sigmoid" (a score per expert) or "softmax" (over all router outputs). The last `identity` router outputs
    (beyond `experts`) stand for experts that return their input. `groups` > 0: the router outputs form that many equal
    groups of neighbours, a group scores as its best choice score, and only members of the best `keep` groups can be chosen.
    `act`: "relu2" (down(relu(up x)^2)), "clamp_glu" (g = min(gate x, limit), u = clamp(up x, -limit, limit),
    down(g sigmoid(1.702 g) (u + 1))) or "silu_glu" (down(silu(gate x) * (up x))). `router` "topk_softmax": the `top` largest
    logits are chosen and weighted by the softmax over the chosen logits only (no correction tensor)."""
    experts: int
    top: int
    ff: int
    scale: float = 1.0
    shared_ff: int = 0
    router: str = "sigmoid"
    identity: int = 0
    groups: int = 0
    keep: int = 0
    act: str = "relu2"
    limit: float = 0.0

    @property
    def outputs(self) -> int:
        """Rows of the router matrix."""
        return self.experts + self.identity


@dataclass
class MaskedAttnConfig:
    """Softmax attention over paged keys and values with per-head q/k RMS norm (one weight of `dim` channels shared by the
    heads), rotary positions on the first rot.dims channels of a head (`rot_pairs`: channel 2i turns with 2i+1, else i with
    i + dims/2), a sliding window (row i sees j with 0 <= i - j < window; 0: none), `value_keys`: the values are the keys
    as projected, before norm and rotation (no value projection), `gate`: "none", "head" or "channel" (sigmoid of a
    projection of the mixer's input, applied before the output projection), `sink`: a zero-logit term in the denominator."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: int
    scale: float
    rot: RotaryConfig
    rot_pairs: bool = True
    value_keys: bool = True
    gate: str = "channel"
    sink: bool = False
    unit_norm: bool = False   # q and k heads are divided by their rms without a weight (no q.norm / k.norm tensors)
    temp: bool = False        # a learned factor per query head on the scores (tensor `temp`)
    v_mix: bool = False       # the cached values are (1 - vmix) v + vmix v_first, v_first = the first such layer's values of the token

    @property
    def gate_rows(self) -> int:
        return {"none": 0, "head": self.heads, "channel": self.heads * self.vdim}[self.gate]


@dataclass
class DeltaConfig:
    """Gated delta rule with a decay per head and key channel: q, k (kv_heads x dim) and v (heads x vdim) pass a causal
    convolution of `conv` taps and silu; q and k become unit vectors per head (q also times dim^-1/2); per head
    S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q with beta = sigmoid(b x) and
    g = exp(-exp(A_log) softplus(a2 (a1 x) + dt_bias)); each head's o is brought to unit rms, times a weight of vdim channels,
    times sigmoid(g2 (g1 x)). The bottleneck ranks come from the tensors' shapes when 0."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int = 4
    rank_a: int = 0
    rank_g: int = 0

    @property
    def conv_channels(self) -> int:
        return 2 * self.kv_heads * self.dim + self.heads * self.vdim


@dataclass
class SeqLayerConfig:
    type: str                      # "mamba2" | "parallel" | "retention" | "latent_attention" | "attention" | "channel_delta"
    ssd: SsdMixerConfig = None
    left: ChunkAttnConfig = None
    right: GlaConfig = None
    ff: int = 0                    # 0 = the layer has no dense feed-forward
    retention: RetentionConfig = None
    latent: LatentAttnConfig = None
    moe: MoeConfig = None          # routed feed-forward instead of the dense one
    attn: MaskedAttnConfig = None  # type "attention"
    delta: DeltaConfig = None      # type "channel_delta"
    weights_of: int = -1           # >= 0: the layer owns no tensors and runs with that layer's (cache and state are its own)


# What an architecture name fixes (everything else comes from config.json): the residual block form, whether the stored
# norm weights are centred on zero (the applied weight is 1 + w), and the position term of the embedding.
SEQ_FAMILIES = {
    "Bimopel": dict(block="postnorm", norm_offset=0.0, positions="sinusoid"),
    "Kedelorn": dict(block="prenorm_hc", norm_offset=1.0, positions=None),
    # parallel blocks behind one Dynamic-Tanh norm; attention whose values are the un-normed keys, pair-interleaved rotary
    # positions, a gate per channel; two-matrix gelu feed-forward; softmax router, clamped gated experts
    "Dibedra": dict(block="parallel", norm_offset=0.0, positions=None, norm="dyt", dense="mlp", router="softmax", expert="clamp_glu",
                    attention=dict(rot_pairs=True, value_keys=True, gate="channel", sink=False)),
    # sublayers read the residual stream itself (the mixer through a short convolution over time) and pass an RMS norm with ONE
    # number as its weight on their way back into it; delta-rule, attention and latent-attention mixers; two-matrix gelu
    # feed-forward; experts chosen by logit, weighted by the softmax over the chosen logits, gated silu experts
    "Lugizen": dict(block="branchnorm", norm_offset=0.0, positions=None, norm_scalar=True, dense="mlp", router="topk_softmax",
                    expert="silu_glu",
                    attention=dict(rot_pairs=False, value_keys=False, gate="none", sink=False, unit_norm=True, temp=True),
                    latent=dict(q_latent=True, gate=False, sink=False)),
}


@dataclass
class SeqModelConfig:
    architecture: str
    vocab: int
    width: int
    layers: list
    eps: float = 1e-5
    alpha: float = 1.0
    embed_scale: float = 1.0
    logit_softcap: float = 0.0
    eos_token_id: int = -1         # none unless config.json names one
    block: str = "postnorm"        # "postnorm" | "prenorm_hc" (pre-norm sublayers on `streams` residual streams) | "parallel" |
                                   # "branchnorm" (x <- x + norm(sublayer(x)); the mixer reads x + conv(x) when canon_taps > 0)
    canon_taps: int = 0            # taps of the causal convolution over time in front of every mixer (tensor l<i>.canon1 [width, taps])
    norm_scalar: bool = False      # a norm's weight is ONE number (tensors of one element)
    norm: str = "rms"              # "rms" | "dyt" (tanh(alpha x) w + b; tensors <name>, <name>.b, <name>.alpha)
    dense: str = "glu"             # dense feed-forward: "glu" (gelu_tanh(gate) * up) | "mlp" (gelu_tanh(up))
    logit_scale: float = 1.0
    streams: int = 1
    norm_offset: float = 0.0       # added to every stored layer-norm weight (1.0: weights stored around zero)
    positions: str = "sinusoid"    # position term of the embedding, or None

    @staticmethod
    def from_json(d: dict) -> "SeqModelConfig":
        """config.json of a hybrid sequence model: `layers` lists each layer's `type`, its mixer's sizes and its `mlp`."""
        arch = d.get("architecture", "Bimopel")
        if arch not in SEQ_FAMILIES:
            raise NotImplementedError(f"architecture {arch!r} is not a hybrid sequence model (known: {sorted(SEQ_FAMILIES)})")
        fam = SEQ_FAMILIES[arch]
        layers = []
        for i, L in enumerate(d["layers"]):
            mx, mlp = L["mixer"], L.get("mlp")
            ff, moe = 0, None
            if mlp is not None:
                kind = mlp.get("kind", "moe" if "router" in mlp else "dense")
                if kind == "dense":
                    ff = int(mlp["ff"])
                elif kind == "moe":
                    r, sh, gr = mlp["router"], mlp.get("shared"), mlp["router"].get("groups")
                    moe = MoeConfig(experts=int(r["experts"]), top=int(r["top"]), ff=int(mlp["expert"]["ff"]),
                                    scale=float(r.get("scale", 1.0)), shared_ff=int(sh["ff"]) if sh else 0,
                                    router=fam.get("router", "sigmoid"), identity=int(r.get("identity", 0)),
                                    groups=int(gr["count"]) if gr else 0, keep=int(gr["keep"]) if gr else 0,
                                    act=fam.get("expert", "relu2"), limit=float(mlp["expert"].get("limit", 0.0)))
                else:
                    raise NotImplementedError(f"layer {i}: feed-forward kind {kind!r} is not supported")
            share = L.get("weights_of")
            if share is not None:        # follow the reference to the layer that owns the tensors
                seen = {i}
                share = int(share)
                while True:
                    if not 0 <= share < len(d["layers"]) or share in seen:
                        raise ValueError(f"layer {i}: weights_of must lead to a layer that owns its tensors")
                    nxt = d["layers"][share].get("weights_of")
                    if nxt is None:
                        break
                    seen.add(share)
                    share = int(nxt)
            if L["type"] == "attention":
                if "attention" not in fam:
                    raise NotImplementedError(f"layer {i}: {arch} has no mixer of type 'attention'")
                rot = RotaryConfig.from_json(mx["rot"]) if mx.get("rot") else RotaryConfig(0, 10000.0)
                layers.append(SeqLayerConfig("attention", ff=ff, moe=moe, weights_of=-1 if share is None else share, attn=MaskedAttnConfig(
                    heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])), dim=int(mx["dim"]),
                    vdim=int(mx.get("vdim", mx["dim"])), window=int((mx.get("mask") or {}).get("size", 0)),
                    scale=float(mx.get("scale", float(mx["dim"]) ** -0.5)), rot=rot, v_mix=bool(mx.get("v_mix", False)), **fam["attention"])))
            elif L["type"] == "channel_delta":
                layers.append(SeqLayerConfig("channel_delta", ff=ff, moe=moe, delta=DeltaConfig(
                    heads=int(mx["heads"]), kv_heads=int(mx.get("kv_heads", mx["heads"])), dim=int(mx["dim"]),
                    vdim=int(mx.get("vdim", mx["dim"])), conv=int(mx.get("conv", 4)), rank_a=int(mx.get("decay_rank", 0)),
                    rank_g=int(mx.get("gate_rank", 0)))))
            elif L["type"] == "retention":
                rot = RotaryConfig.from_json(mx["rot"]) if mx.get("rot") else RotaryConfig(0, 10000.0)
                layers.append(SeqLayerConfig("retention", ff=ff, moe=moe, retention=RetentionConfig(
                    heads=int(mx["heads"]), dim=int(mx["dim"]), vdim=int(mx.get("vdim", mx["dim"])),
                    decay=[float(x) for x in mx["decay"]], rot=rot)))
            elif L["type"] == "latent_attention":
                src = mx.get("kv_from")
                lf = fam.get("latent", {})
                layers.append(SeqLayerConfig("latent_attention", ff=ff, moe=moe, latent=LatentAttnConfig(
                    heads=int(mx["heads"]), dim=int(mx["dim"]), rot_dim=int(mx["rot_dim"]), vdim=int(mx.get("vdim", mx["dim"])),
                    kv_rank=int(mx["kv_rank"]), scale=float(mx["scale"]), rot=RotaryConfig.from_json(mx["rot"], int(mx["rot_dim"])),
                    kv_from=-1 if src is None else int(src), q_rank=int(mx.get("q_rank", 0)) if lf.get("q_latent") else 0,
                    window=int((mx.get("mask") or {}).get("size", 0)), gate=lf.get("gate", True), sink=lf.get("sink", True))))
            elif L["type"] == "mamba2":
                layers.append(SeqLayerConfig("mamba2", ssd=SsdMixerConfig(
                    heads=int(mx["heads"]), vdim=int(mx["vdim"]), state=int(mx["state"]), groups=int(mx.get("groups", 1)),
                    conv=int(mx.get("conv", 4)), norm_groups=int(mx.get("norm_groups", 1))), ff=ff, moe=moe))
            elif L["type"] == "parallel":
                l, r = mx["left"], mx["right"]
                left = ChunkAttnConfig(heads=int(l["heads"]), kv_heads=int(l.get("kv_heads", l["heads"])), dim=int(l["dim"]),
                                       vdim=int(l.get("vdim", l["dim"])), chunk=int((l.get("mask") or {}).get("size", 0)),
                                       scale=float(l.get("scale", float(l["dim"]) ** -0.5)))
                right = GlaConfig(heads=int(r["heads"]), dim=int(r["dim"]), vdim=int(r.get("vdim", r["dim"])),
                                  tau=float(r.get("tau", 1.0)))
                layers.append(SeqLayerConfig("parallel", left=left, right=right, ff=ff, moe=moe))
            else:
                raise NotImplementedError(f"layer {i}: mixer type {L['type']!r} is not supported")
        return SeqModelConfig(
            architecture=arch, vocab=int(d["vocab"]), width=int(d["width"]), layers=layers,
            eps=float((d.get("norm") or {}).get("eps", 1e-5)), alpha=float(d.get("postln_alpha", 1.0)),
            embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)), logit_softcap=float(d.get("logit_softcap") or 0.0),
            eos_token_id=int(d.get("eos_token_id", -1)), block=fam["block"], streams=int(d.get("streams", 1)),
            norm_offset=fam["norm_offset"], positions=fam["positions"], norm=fam.get("norm", "rms"), dense=fam.get("dense", "glu"),
            logit_scale=float(d.get("logit_scale", 1.0)), canon_taps=int((d.get("canon") or {}).get("taps", 0)),
            norm_scalar=bool(fam.get("norm_scalar", False)))

    def to_json(self) -> dict:
        """The inverse of from_json (used to write synthetic checkpoints)."""
        out = []
        for L in self.layers:
            if L.type == "mamba2":
                s = L.ssd
                mx = dict(heads=s.heads, vdim=s.vdim, state=s.state, groups=s.groups, conv=s.conv, norm_groups=s.norm_groups)
            elif L.type == "retention":
                t = L.retention
                mx = dict(heads=t.heads, dim=t.dim, vdim=t.vdim, decay=list(t.decay), rot=t.rot.to_json())
            elif L.type == "latent_attention":
                a = L.latent
                mx = dict(heads=a.heads, dim=a.dim, rot_dim=a.rot_dim, vdim=a.vdim, kv_rank=a.kv_rank, scale=a.scale, rot=a.rot.to_json())
                if a.kv_from >= 0:
                    mx["kv_from"] = a.kv_from
                if a.q_rank:
                    mx["q_rank"] = a.q_rank
                if a.window:
                    mx["mask"] = dict(size=a.window)
            elif L.type == "attention":
                a = L.attn
                mx = dict(heads=a.heads, kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim, scale=a.scale, rot=a.rot.to_json())
                if a.window:
                    mx["mask"] = dict(size=a.window)
                if a.v_mix:
                    mx["v_mix"] = True
            elif L.type == "channel_delta":
                t = L.delta
                mx = dict(heads=t.heads, kv_heads=t.kv_heads, dim=t.dim, vdim=t.vdim, conv=t.conv)
                if t.rank_a:
                    mx["decay_rank"] = t.rank_a
                if t.rank_g:
                    mx["gate_rank"] = t.rank_g
            else:
                l, r = L.left, L.right
                mx = dict(left=dict(heads=l.heads, kv_heads=l.kv_heads, dim=l.dim, vdim=l.vdim, mask=dict(size=l.chunk), scale=l.scale),
                          right=dict(heads=r.heads, dim=r.dim, vdim=r.vdim, tau=r.tau))
            mlp = dict(ff=L.ff, kind="dense") if L.ff else None
            if L.moe:
                e = L.moe
                mlp = dict(kind="moe", expert=dict(ff=e.ff), router=dict(experts=e.experts, top=e.top, scale=e.scale))
                if e.shared_ff:
                    mlp["shared"] = dict(ff=e.shared_ff)
                if e.act == "clamp_glu":
                    mlp["expert"]["limit"] = e.limit
                if e.act != "relu2":
                    del mlp["router"]["scale"]
                if e.identity:
                    mlp["router"]["identity"] = e.identity
                if e.groups:
                    mlp["router"]["groups"] = dict(count=e.groups, keep=e.keep)
            out.append(dict(type=L.type, mixer=mx, mlp=mlp))
            if L.weights_of >= 0:
                out[-1]["weights_of"] = L.weights_of
        if self.block == "branchnorm":
            out_d = dict(architecture=self.architecture, vocab=self.vocab, width=self.width, layers=out, norm=dict(eps=self.eps))
            if self.canon_taps:
                out_d["canon"] = dict(taps=self.canon_taps)
            return out_d
        if self.block == "parallel":
            return dict(architecture=self.architecture, vocab=self.vocab, width=self.width, layers=out, norm=dict(eps=self.eps),
                        logit_scale=self.logit_scale)
        if self.block == "prenorm_hc":
            return dict(architecture=self.architecture, vocab=self.vocab, width=self.width, streams=self.streams, layers=out,
                        norm=dict(eps=self.eps))
        return dict(architecture=self.architecture, vocab=self.vocab, width=self.width, layers=out, norm=dict(eps=self.eps),
                    postln_alpha=self.alpha, embedding=dict(scale=self.embed_scale), logit_softcap=self.logit_softcap)

    def validate(self) -> None:
        if self.width < 1 or self.vocab < 1:
            raise ValueError("width and vocab must be positive")
        if self.block == "prenorm_hc" and not 1 <= self.streams <= 8:
            raise ValueError("1 to 8 residual streams")
        if not 0 <= self.canon_taps <= 8 or (self.canon_taps and self.block != "branchnorm"):
            raise ValueError("a convolution of 1 to 8 taps in front of the mixers is served in blocks normed on the sublayer's output")
        for i, L in enumerate(self.layers):
            if L.moe and not (1 <= L.moe.top <= L.moe.outputs <= 512 and L.moe.experts >= 1 and L.moe.identity >= 0):
                raise ValueError(f"layer {i}: unsupported router sizes {L.moe}")
            if L.moe and L.moe.groups and (L.moe.outputs % L.moe.groups or not 1 <= L.moe.keep <= L.moe.groups or
                                           L.moe.keep * (L.moe.outputs // L.moe.groups) < L.moe.top):
                raise ValueError(f"layer {i}: the kept groups must be equal groups that hold at least `top` experts: {L.moe}")
            if L.moe and (L.moe.identity or L.moe.act == "clamp_glu") and L.moe.shared_ff:
                raise ValueError(f"layer {i}: identity experts and a shared expert do not combine")
            if L.weights_of >= 0 and self.block != "parallel":
                raise ValueError(f"layer {i}: shared layer weights are served in parallel blocks only")
            if L.moe and L.moe.router == "topk_softmax" and (L.moe.identity or L.moe.groups or L.moe.shared_ff):
                raise ValueError(f"layer {i}: weights over the chosen logits combine with neither identity experts, groups nor a shared expert")
            if L.type == "channel_delta":
                t = L.delta
                if t.heads < 1 or t.kv_heads < 1 or t.heads % t.kv_heads or not 1 <= t.dim <= 512 or t.vdim < 1 or not 1 <= t.conv <= 8:
                    raise ValueError(f"layer {i}: unsupported delta-rule sizes {t}")
                continue
            if L.type == "attention":
                a = L.attn
                if self.block not in ("parallel", "branchnorm"):
                    raise ValueError(f"layer {i}: the attention mixer is served in parallel blocks and in blocks normed on the sublayer's output")
                if a.v_mix:
                    first = next(x.attn for x in self.layers if x.type == "attention" and x.attn.v_mix)
                    if a.value_keys or (first.kv_heads, first.vdim) != (a.kv_heads, a.vdim):
                        raise ValueError(f"layer {i}: layers that mix values share the shape of their projected values")
                if a.heads < 1 or a.kv_heads < 1 or a.heads % a.kv_heads or a.dim < 1 or a.window < 0 or a.rot.dims % 2 or \
                        a.rot.dims > a.dim or (a.value_keys and a.vdim != a.dim):
                    raise ValueError(f"layer {i}: unsupported attention sizes {a}")
                continue
            if L.type == "mamba2":
                s = L.ssd
                if s.heads % s.groups or s.inner % s.norm_groups or not 1 <= s.conv <= 8 or s.state > 512:
                    raise ValueError(f"layer {i}: unsupported state-space sizes {s}")
            elif L.type == "retention":
                t = L.retention
                if len(t.decay) != t.heads or t.dim > 512 or t.rot.dims % 2 or t.rot.dims > t.dim or \
                        any(not 0.0 < x <= 1.0 for x in t.decay):
                    raise ValueError(f"layer {i}: unsupported retention sizes {t}")
            elif L.type == "latent_attention":
                a = L.latent
                if a.rot.dims != a.rot_dim or a.rot_dim % 2 or a.rot_dim < 2:
                    raise ValueError(f"layer {i}: the rotated part of a latent-attention head is rot_dim = rot.dims (even) channels")
                if a.q_rank < 0 or a.window < 0:
                    raise ValueError(f"layer {i}: unsupported latent-attention sizes {a}")
                if a.kv_from >= 0:
                    o = self.layers[a.kv_from] if a.kv_from < i else None
                    if o is None or o.type != "latent_attention" or o.latent.kv_from >= 0 or \
                            (o.latent.kv_rank, o.latent.rot_dim, o.latent.rot) != (a.kv_rank, a.rot_dim, a.rot):
                        raise ValueError(f"layer {i}: kv_from must name an earlier latent-attention layer with its own cache and the same geometry")
            else:
                if L.left.heads % L.left.kv_heads or L.right.dim > 512:
                    raise ValueError(f"layer {i}: unsupported attention sizes")
