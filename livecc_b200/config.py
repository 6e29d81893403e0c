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
class SeqLayerConfig:
    type: str                      # "mamba2" | "parallel"
    ssd: SsdMixerConfig = None
    left: ChunkAttnConfig = None
    right: GlaConfig = None
    ff: int = 0                    # 0 = the layer has no feed-forward


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

    @staticmethod
    def from_json(d: dict) -> "SeqModelConfig":
        """config.json of a hybrid sequence model: `layers` lists each layer's `type`, its mixer's sizes and its `mlp`."""
        layers = []
        for i, L in enumerate(d["layers"]):
            mx, mlp = L["mixer"], L.get("mlp")
            ff = 0
            if mlp is not None:
                if mlp.get("kind", "dense") != "dense":
                    raise NotImplementedError(f"layer {i}: feed-forward kind {mlp.get('kind')!r} is not supported")
                ff = int(mlp["ff"])
            if L["type"] == "mamba2":
                layers.append(SeqLayerConfig("mamba2", ssd=SsdMixerConfig(
                    heads=int(mx["heads"]), vdim=int(mx["vdim"]), state=int(mx["state"]), groups=int(mx.get("groups", 1)),
                    conv=int(mx.get("conv", 4)), norm_groups=int(mx.get("norm_groups", 1))), ff=ff))
            elif L["type"] == "parallel":
                l, r = mx["left"], mx["right"]
                left = ChunkAttnConfig(heads=int(l["heads"]), kv_heads=int(l.get("kv_heads", l["heads"])), dim=int(l["dim"]),
                                       vdim=int(l.get("vdim", l["dim"])), chunk=int((l.get("mask") or {}).get("size", 0)),
                                       scale=float(l.get("scale", float(l["dim"]) ** -0.5)))
                right = GlaConfig(heads=int(r["heads"]), dim=int(r["dim"]), vdim=int(r.get("vdim", r["dim"])),
                                  tau=float(r.get("tau", 1.0)))
                layers.append(SeqLayerConfig("parallel", left=left, right=right, ff=ff))
            else:
                raise NotImplementedError(f"layer {i}: mixer type {L['type']!r} is not supported")
        return SeqModelConfig(
            architecture=d.get("architecture", "Bimopel"), vocab=int(d["vocab"]), width=int(d["width"]), layers=layers,
            eps=float((d.get("norm") or {}).get("eps", 1e-5)), alpha=float(d.get("postln_alpha", 1.0)),
            embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)), logit_softcap=float(d.get("logit_softcap") or 0.0),
            eos_token_id=int(d.get("eos_token_id", -1)))

    def to_json(self) -> dict:
        """The inverse of from_json (used to write synthetic checkpoints)."""
        out = []
        for L in self.layers:
            if L.type == "mamba2":
                s = L.ssd
                mx = dict(heads=s.heads, vdim=s.vdim, state=s.state, groups=s.groups, conv=s.conv, norm_groups=s.norm_groups)
            else:
                l, r = L.left, L.right
                mx = dict(left=dict(heads=l.heads, kv_heads=l.kv_heads, dim=l.dim, vdim=l.vdim, mask=dict(size=l.chunk), scale=l.scale),
                          right=dict(heads=r.heads, dim=r.dim, vdim=r.vdim, tau=r.tau))
            out.append(dict(type=L.type, mixer=mx, mlp=dict(ff=L.ff, kind="dense") if L.ff else None))
        return dict(architecture=self.architecture, vocab=self.vocab, width=self.width, layers=out, norm=dict(eps=self.eps),
                    postln_alpha=self.alpha, embedding=dict(scale=self.embed_scale), logit_softcap=self.logit_softcap)

    def validate(self) -> None:
        if self.width < 1 or self.vocab < 1:
            raise ValueError("width and vocab must be positive")
        for i, L in enumerate(self.layers):
            if L.type == "mamba2":
                s = L.ssd
                if s.heads % s.groups or s.inner % s.norm_groups or not 1 <= s.conv <= 8 or s.state > 512:
                    raise ValueError(f"layer {i}: unsupported state-space sizes {s}")
            else:
                if L.left.heads % L.left.kv_heads or L.right.dim > 512:
                    raise ValueError(f"layer {i}: unsupported attention sizes")
