"""The Lafanex decoder's configuration, read from its own config.json keys.

Lafanex is a pre-norm decoder over several 32-bit residual streams (hyper-connections: ``streams`` copies of the residual,
each sublayer reads a weighted sum of them and writes back through a mixing matrix), root-mean-square norms whose weights
are stored around zero, and logits against the embedding table. ``layers`` lists its layers: each names its mixer by
``type`` (``attention``: grouped-query causal attention with values of a size of their own, a rotation of interleaved
pairs, unit-root-mean-square queries and keys and one added to the softmax's denominator; ``mamba1``: a short convolution
and the selective scan) with the mixer's sizes under ``mixer``, and its feed-forward under ``mlp`` (``dense``: a gated one
with the tanh form of GELU; ``moe``: routed experts with softmax scores, a correction for the choice, identity experts
and a gated shared expert; null: none). ``loop`` names a range of layers that runs several times in a row with the same
weights; every pass keeps a cache or state of its own. Tensor names: ``embed``, ``l<i>.norm1`` / ``.norm2``,
``l<i>.hc1.*`` / ``.hc2.*``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``. No size and no constant that config.json
gives stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .reader import ConfigError, ConfigReader
from .spec import (BlockSpec, ConnectionSpec, GatedMlpSpec, Mamba1Spec, ModelSpec, NormSpec, PositionSpec, RoutedMlpSpec, RunEntry,
                   SinkAttentionSpec)

ARCHITECTURE = "Lafanex"
ROUTED_GATE_SLOPE = 1.702      # the design's constant inside the experts' activation: g sigmoid(1.702 g) (u + 1)


@dataclass(frozen=True)
class LafanexLayer:
    type: str
    mixer: dict            # the mixer's sizes and constants, checked and typed
    mlp: dict | None


def _positive_float(r: ConfigReader, key: str) -> float:
    v = r.opt_float(key)
    if v is None or not v > 0:
        raise ConfigError(f"{r.source}: key '{key}' must be a positive number")
    return v


@dataclass
class LafanexConfig:
    vocab: int
    width: int
    eps: float
    streams: int | None            # None: one residual and plain sums
    layers: tuple
    loop: tuple | None             # (start, stop, times)
    tie_word_embeddings: bool = True
    warnings: list = field(default_factory=list)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_reader(cls, c: ConfigReader) -> "LafanexConfig":
        vocab, width = c.positive_int("vocab"), c.positive_int("width")
        norm = c.opt_object("norm")
        if norm is None:
            raise ConfigError(f"{c.source}: key 'norm.eps' must be a positive number")
        eps = _positive_float(norm, "eps")
        streams = c.positive_int("streams") if c.has("streams") and c.raw("streams") is not None else None
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
            if kind == "attention":
                mixer = cls._read_attention(m)
            elif kind == "mamba1":
                mixer = cls._read_mamba(m)
            else:
                raise ConfigError(f"{lr.source}: key 'type' is {kind!r}; the design has attention and mamba1 mixers")
            layers.append(LafanexLayer(kind, mixer, cls._read_mlp(lr.opt_object("mlp"))))
        loop = None
        lp = c.opt_object("loop")
        if lp is not None:
            start, stop, times = lp.opt_int("start"), lp.opt_int("stop"), lp.positive_int("times")
            if start is None or stop is None or not 0 <= start <= stop <= len(layers):
                raise ConfigError(f"{lp.source}: 'start' and 'stop' must bound a range of the {len(layers)} layers")
            loop = (start, stop, times)
        return cls(vocab=vocab, width=width, eps=eps, streams=streams, layers=tuple(layers), loop=loop)

    @staticmethod
    def _read_attention(m: ConfigReader) -> dict:
        out = {k: m.positive_int(k) for k in ("heads", "kv_heads", "dim", "vdim")}
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"{m.source}: {out['heads']} heads are not a multiple of {out['kv_heads']} kv_heads")
        out["scale"] = _positive_float(m, "scale")
        rot = m.opt_object("rot")
        if rot is None:
            raise ConfigError(f"{m.source}: key 'rot' is absent")
        out["rot_dims"], out["rot_base"] = rot.positive_int("dims"), _positive_float(rot, "base")
        if out["rot_dims"] % 2 or out["rot_dims"] > out["dim"]:
            raise ConfigError(f"{rot.source}: key 'dims' is {out['rot_dims']}; it must be even and at most dim {out['dim']}")
        return out

    @staticmethod
    def _read_mamba(m: ConfigReader) -> dict:
        return {k: m.positive_int(k) for k in ("inner", "state", "dt_rank", "conv")}

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
            identity = router.opt_int("identity") or 0
            scale = router.opt_float("scale")
            out = {"kind": "moe", "experts": router.positive_int("experts"), "top": router.positive_int("top"), "identity": identity,
                   "scale": 1.0 if scale is None else scale, "ff": expert.positive_int("ff"), "limit": _positive_float(expert, "limit"),
                   "shared_ff": shared.positive_int("ff") if shared is not None else 0,
                   "shared_limit": _positive_float(shared, "limit") if shared is not None else 0.0}
            if identity < 0:
                raise ConfigError(f"{router.source}: key 'identity' is {identity}; it cannot be negative")
            if out["top"] > out["experts"] + identity:
                raise ConfigError(f"{router.source}: top {out['top']} is more than the {out['experts']} experts and {identity} identity experts")
            return out
        raise ConfigError(f"{f.source}: key 'kind' is {kind!r}; the design has dense and moe feed-forwards")

    @classmethod
    def from_dict(cls, values: dict, source: str = "config") -> "LafanexConfig":
        return cls.from_reader(ConfigReader(values, source))

    # ------------------------------------------------------------------ the model as parts
    def layer_order(self) -> list:
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def to_spec(self, tied: bool | None = None) -> ModelSpec:
        W = self.width
        norm = NormSpec(size=W, eps=self.eps, kind="rms_norm", weight_offset=1.0)
        connection = ConnectionSpec(streams=self.streams or 1, learned=self.streams is not None)
        names: dict = {"embed": {"table": ("embed",)}, "final_norm": {"weight": ("final.norm",)}}
        blocks, unused = [], []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer.mixer
            if layer.type == "attention":
                mixer = SinkAttentionSpec(hidden=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], v_dim=m["vdim"],
                                          scale=m["scale"], sink=True, unit_norm_eps=self.eps,
                                          position=PositionSpec(kind="rope_interleaved", rotary_dim=m["rot_dims"], theta=m["rot_base"]))
                mix_names = {"qkv": (p + "mix.q", p + "mix.k", p + "mix.v"), "out": (p + "mix.o",)}
            else:
                mixer = Mamba1Spec(hidden=W, inner=m["inner"], state=m["state"], dt_rank=m["dt_rank"], conv_taps=m["conv"])
                mix_names = {"in": (p + "mix.in",), "conv": (p + "mix.conv",), "conv_bias": (p + "mix.conv.b",), "x": (p + "mix.x",),
                             "dt": (p + "mix.dt",), "dt_bias": (p + "mix.dt.b",), "A_log": (p + "mix.A_log",), "D": (p + "mix.D",),
                             "out": (p + "mix.o",)}
            f = layer.mlp
            if f is None:
                ff = None
            elif f["kind"] == "dense":
                ff = GatedMlpSpec(hidden=W, intermediate=f["ff"], activation="gelu_tanh")
                names[f"blocks.{i}.feed_forward"] = {"gate_up": (p + "mlp.gate", p + "mlp.up"), "down": (p + "mlp.down",)}
            else:
                ff = RoutedMlpSpec(hidden=W, experts=f["experts"], top=f["top"], expert_intermediate=f["ff"], shared_intermediate=f["shared_ff"],
                                   activation="clamped_swish", score="softmax", renormalize=False, weight_on="output", correction=True,
                                   route_scale=f["scale"], identity_experts=f["identity"], limit=f["limit"], shared_limit=f["shared_limit"],
                                   shared_gate=bool(f["shared_ff"]))
                E = range(f["experts"])
                ff_names = {"router": (p + "mlp.router",), "correction": (p + "mlp.correction",),
                            "gate": tuple(f"{p}mlp.e{e}.gate" for e in E), "up": tuple(f"{p}mlp.e{e}.up" for e in E),
                            "down": tuple(f"{p}mlp.e{e}.down" for e in E)}
                if f["shared_ff"]:
                    ff_names.update({"shared_gate_up": (p + "mlp.shared.gate", p + "mlp.shared.up"), "shared_down": (p + "mlp.shared.down",),
                                     "shared_gate": (p + "mlp.shared.sg",)})
                names[f"blocks.{i}.feed_forward"] = ff_names
            blocks.append(BlockSpec(mixer=mixer, feed_forward=ff, input_norm=norm, post_mixer_norm=norm if ff is not None else None,
                                    kind="pre_norm_streams", connection=connection))
            names[f"blocks.{i}.input_norm"] = {"weight": (p + "norm1",)}
            names[f"blocks.{i}.mixer"] = mix_names
            if connection.learned:
                names[f"blocks.{i}.mixer_connection"] = {"in": (p + "hc1.in",), "out": (p + "hc1.out",), "mix": (p + "hc1.mix",)}
            if ff is not None:
                names[f"blocks.{i}.post_mixer_norm"] = {"weight": (p + "norm2",)}
                if connection.learned:
                    names[f"blocks.{i}.feed_forward_connection"] = {"in": (p + "hc2.in",), "out": (p + "hc2.out",), "mix": (p + "hc2.mix",)}
            else:       # a layer without a feed-forward applies neither its second norm nor its second connection
                unused += [p + "norm2", p + "hc2.in", p + "hc2.out", p + "hc2.mix"]
        # every pass of the looped range is a run of its own: the same weights, a cache or state of its own
        schedule = tuple(RunEntry(block=i) for i in self.layer_order())
        return ModelSpec(architecture=ARCHITECTURE, hidden=W, vocab=self.vocab, blocks=tuple(blocks), schedule=schedule, final_norm=norm,
                         tie_embeddings=True, max_positions=0, stop_token_ids=(), stored_dtype="bfloat16", ignorable_tensors=tuple(unused),
                         weight_names=names)
