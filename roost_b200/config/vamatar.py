"""The Vamatar decoder's configuration, read from its own config.json keys.

Vamatar is a pre-norm decoder with a 32-bit residual stream, layer norms with bias, a scaled embedding and tanh-capped
logits. ``layers`` lists its layers: each names its mixer by ``type`` (``latent_attention``: keys and values made per
head from a cached latent and one shared rotated key part, under a sliding window, possibly reading the latent of an
earlier layer through ``kv_from``; ``mamba2``: a short convolution and the Mamba-2 recurrence) with the mixer's sizes
under ``mixer``, and its feed-forward under ``mlp`` (``dense``: one gated feed-forward; ``moe``: routed experts with
sigmoid scores that multiply the chosen experts' input, and a shared expert; null: none). Tensor names: ``embed``,
``l<i>.norm1`` / ``.norm2`` (bias: the same name with ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
No size and no constant that config.json gives stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .reader import ConfigError, ConfigReader
from .spec import (BlockSpec, CappedHeadSpec, GatedMlpSpec, HeadSpec, LatentAttentionSpec, Mamba2Spec, ModelSpec, NormSpec, PositionSpec,
                   RoutedMlpSpec, RunEntry, ScaledEmbeddingSpec)

ARCHITECTURE = "Vamatar"


@dataclass(frozen=True)
class VamatarLayer:
    type: str
    mixer: dict            # the mixer's sizes and constants, checked and typed
    mlp: dict | None


@dataclass
class VamatarConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_softcap: float | None
    layers: tuple
    tie_word_embeddings: bool = False
    warnings: list = field(default_factory=list)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_reader(cls, c: ConfigReader) -> "VamatarConfig":
        vocab, width = c.positive_int("vocab"), c.positive_int("width")
        norm = c.opt_object("norm")
        eps = norm.opt_float("eps") if norm is not None else None
        if eps is None or eps <= 0:
            raise ConfigError(f"{c.source}: key 'norm.eps' must be a positive number")
        emb = c.opt_object("embedding")
        scale = emb.opt_float("scale") if emb is not None else None
        cap = c.opt_float("logit_softcap")
        if cap is not None and cap <= 0:
            raise ConfigError(f"{c.source}: key 'logit_softcap' is {cap}; it must be positive")
        raw = c.raw("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError(f"{c.source}: key 'layers' must be a non-empty list")
        layers = []
        for i, item in enumerate(raw):
            lr = ConfigReader(item, f"{c.source}: layers[{i}]")
            kind = lr.opt_str("type")
            m = lr.opt_object("mixer")
            if m is None:
                raise ConfigError(f"{lr.source}: key 'mixer' is absent")
            if kind == "latent_attention":
                mixer = cls._read_latent(m, i, layers)
            elif kind == "mamba2":
                mixer = cls._read_mamba(m)
            else:
                raise ConfigError(f"{lr.source}: key 'type' is {kind!r}; the design has latent_attention and mamba2 mixers")
            layers.append(VamatarLayer(kind, mixer, cls._read_mlp(lr.opt_object("mlp"))))
        return cls(vocab=vocab, width=width, eps=eps, embedding_scale=1.0 if scale is None else scale, logit_softcap=cap,
                   layers=tuple(layers))

    @staticmethod
    def _read_latent(m: ConfigReader, index: int, before: list) -> dict:
        out = {k: m.positive_int(k) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank")}
        out["scale"] = m.opt_float("scale")
        if out["scale"] is None or out["scale"] <= 0:
            raise ConfigError(f"{m.source}: key 'scale' must be a positive number")
        rot = m.opt_object("rot")
        if rot is None:
            raise ConfigError(f"{m.source}: key 'rot' is absent")
        out["rot_dims"], out["rot_base"] = rot.positive_int("dims"), rot.opt_float("base")
        if out["rot_base"] is None or out["rot_base"] <= 0:
            raise ConfigError(f"{rot.source}: key 'base' must be a positive number")
        if out["rot_dims"] % 2 or out["rot_dims"] > out["rot_dim"]:
            raise ConfigError(f"{rot.source}: key 'dims' is {out['rot_dims']}; it must be even and at most rot_dim {out['rot_dim']}")
        mask = m.opt_object("mask")
        out["window"] = mask.positive_int("size") if mask is not None and mask.has("size") else None
        src = m.opt_int("kv_from")
        out["kv_from"] = src
        if src is not None:
            if not 0 <= src < index or before[src].type != "latent_attention" or before[src].mixer["kv_from"] is not None:
                raise ConfigError(f"{m.source}: key 'kv_from' is {src}; it must name an earlier latent_attention layer that makes its own latent")
            o = before[src].mixer
            for k in ("kv_rank", "rot_dim", "rot_dims", "rot_base"):
                if o[k] != out[k]:
                    raise ConfigError(f"{m.source}: '{k}' is {out[k]} but layer {src}, whose latent it reads, has {o[k]}")
        return out

    @staticmethod
    def _read_mamba(m: ConfigReader) -> dict:
        out = {k: m.positive_int(k) for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups")}
        if out["heads"] % out["groups"]:
            raise ConfigError(f"{m.source}: {out['heads']} heads are not a multiple of {out['groups']} groups")
        if (out["heads"] * out["vdim"]) % out["norm_groups"]:
            raise ConfigError(f"{m.source}: heads x vdim = {out['heads'] * out['vdim']} does not divide into {out['norm_groups']} norm groups")
        return out

    @staticmethod
    def _read_mlp(f: ConfigReader | None) -> dict | None:
        if f is None:
            return None
        kind = f.opt_str("kind")
        if kind == "dense":
            return {"kind": "dense", "ff": f.positive_int("ff")}
        if kind == "moe":
            router, expert, shared = f.opt_object("router"), f.opt_object("expert"), f.opt_object("shared")
            if router is None or expert is None:
                raise ConfigError(f"{f.source}: a moe feed-forward needs 'router' and 'expert'")
            out = {"kind": "moe", "experts": router.positive_int("experts"), "top": router.positive_int("top"),
                   "ff": expert.positive_int("ff"), "shared_ff": shared.positive_int("ff") if shared is not None else 0}
            if out["top"] > out["experts"]:
                raise ConfigError(f"{router.source}: top {out['top']} is more than the {out['experts']} experts")
            return out
        raise ConfigError(f"{f.source}: key 'kind' is {kind!r}; the design has dense and moe feed-forwards")

    @classmethod
    def from_dict(cls, values: dict, source: str = "config") -> "VamatarConfig":
        return cls.from_reader(ConfigReader(values, source))

    # ------------------------------------------------------------------ the model as parts
    def to_spec(self, tied: bool | None = None) -> ModelSpec:
        W = self.width
        norm = NormSpec(size=W, eps=self.eps, kind="layer_norm")
        # a latent cache is kept for the widest window among the layer that makes it and the layers that read it
        keep: dict[int, int | None] = {}
        for i, layer in enumerate(self.layers):
            if layer.type != "latent_attention":
                continue
            owner = i if layer.mixer["kv_from"] is None else layer.mixer["kv_from"]
            w = layer.mixer["window"]
            keep[owner] = w if owner not in keep else (None if w is None or keep[owner] is None else max(w, keep[owner]))
        names: dict = {"embed": {"table": ("embed",)}, "final_norm": {"weight": ("final.norm",), "bias": ("final.norm.b",)},
                       "lm_head": {"weight": ("head",)}}
        blocks, schedule, unused = [], [], []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer.mixer
            if layer.type == "latent_attention":
                owner = i if m["kv_from"] is None else m["kv_from"]
                mixer = LatentAttentionSpec(hidden=W, num_heads=m["heads"], nope_dim=m["dim"], rope_dim=m["rot_dim"], v_dim=m["vdim"],
                                            kv_rank=m["kv_rank"], scale=m["scale"], window=m["window"], cache_window=keep[owner],
                                            own_latent=m["kv_from"] is None, latent_eps=self.eps,
                                            position=PositionSpec(kind="rope_neox", rotary_dim=m["rot_dims"], theta=m["rot_base"]))
                mix_names = {"q": (p + "mix.q",), "uk": (p + "mix.uk",), "uv": (p + "mix.uv",), "out": (p + "mix.o",)}
                if m["kv_from"] is None:
                    mix_names.update({"dkv": (p + "mix.dkv",), "latent_norm": (p + "mix.dkv.norm",)})
                schedule.append(RunEntry(block=i, reads_cache_of=m["kv_from"]))
            else:
                mixer = Mamba2Spec(hidden=W, num_heads=m["heads"], head_dim=m["vdim"], state=m["state"], groups=m["groups"],
                                   conv_taps=m["conv"], norm_groups=m["norm_groups"], eps=self.eps)
                mix_names = {"in": (p + "mix.in",), "conv": (p + "mix.conv",), "conv_bias": (p + "mix.conv.b",), "dt_bias": (p + "mix.dt_bias",),
                             "A_log": (p + "mix.A_log",), "D": (p + "mix.D",), "norm": (p + "mix.norm",), "out": (p + "mix.o",)}
                schedule.append(RunEntry(block=i))
            f = layer.mlp
            if f is None:
                ff = None
            elif f["kind"] == "dense":
                ff = GatedMlpSpec(hidden=W, intermediate=f["ff"], activation="silu")
                names[f"blocks.{i}.feed_forward"] = {"gate_up": (p + "mlp.gate", p + "mlp.up"), "down": (p + "mlp.down",)}
            else:
                ff = RoutedMlpSpec(hidden=W, experts=f["experts"], top=f["top"], expert_intermediate=f["ff"],
                                   shared_intermediate=f["shared_ff"], activation="silu", score="sigmoid", renormalize=False,
                                   weight_on="input")
                E = range(f["experts"])
                ff_names = {"router": (p + "mlp.router",), "gate": tuple(f"{p}mlp.e{e}.gate" for e in E),
                            "up": tuple(f"{p}mlp.e{e}.up" for e in E), "down": tuple(f"{p}mlp.e{e}.down" for e in E)}
                if f["shared_ff"]:
                    ff_names.update({"shared_gate_up": (p + "mlp.shared.gate", p + "mlp.shared.up"), "shared_down": (p + "mlp.shared.down",)})
                names[f"blocks.{i}.feed_forward"] = ff_names
            blocks.append(BlockSpec(mixer=mixer, feed_forward=ff, input_norm=norm, post_mixer_norm=norm if ff is not None else None,
                                    kind="pre_norm_wide"))
            names[f"blocks.{i}.input_norm"] = {"weight": (p + "norm1",), "bias": (p + "norm1.b",)}
            if ff is not None:
                names[f"blocks.{i}.post_mixer_norm"] = {"weight": (p + "norm2",), "bias": (p + "norm2.b",)}
            else:       # a layer without a feed-forward never applies its second norm
                unused += [p + "norm2", p + "norm2.b"]
            names[f"blocks.{i}.mixer"] = mix_names
        head = (CappedHeadSpec(vocab=self.vocab, hidden=W, cap=self.logit_softcap) if self.logit_softcap
                else HeadSpec(vocab=self.vocab, hidden=W))
        return ModelSpec(architecture=ARCHITECTURE, hidden=W, vocab=self.vocab, blocks=tuple(blocks), schedule=tuple(schedule),
                         final_norm=norm, tie_embeddings=False, max_positions=0, stop_token_ids=(), stored_dtype="bfloat16",
                         embedding=ScaledEmbeddingSpec(vocab=self.vocab, hidden=W, scale=self.embedding_scale), head=head,
                         ignorable_tensors=tuple(unused), weight_names=names)
