"""Venidra: a decoder whose layers carry a norm before and after each sublayer, x <- x + norm_b(sublayer(norm(x))), and
whose mixers are either grouped-query softmax attention (query/key and value heads of sizes of their own, a rotate-half
rotation of the heads' first coordinates, q and k divided by their root mean square after the rotation, a chunk mask,
values blended with those of the first blending layer) or attention through low-rank latents (queries through a normed
latent, keys and values from one normed latent per token plus one key part rotated by neighbouring pairs that all heads
share, a sliding window), each followed by a feed-forward gated with the tanh form of GELU, or by none. The embedding is
scaled, the head is the embedding table, the logits are scaled and capped.

config.json keys (every size, and every constant that differs between models of the design):
  architecture "Venidra"; vocab, width; norm.eps; embedding.scale; logit_scale; logit_softcap;
  layers[i] = {type: "attention", mixer: {heads, kv_heads, dim, vdim, scale, rot: {dims, base}, mask: {size}, v_mix}, mlp}
            | {type: "latent_attention", mixer: {heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot: {base, dims},
                                                 mask: {size}}, mlp}
     with mlp = {kind: "dense", ff} | null.
  Left out: kv_heads = heads, vdim = dim, rot = no rotation (attention), rot.dims = rot_dim (latent attention),
  mask = none, v_mix = false, embedding.scale = 1, logit_scale = 1, logit_softcap = none.
Tensors: embed (also the head), final.norm, and per layer l<i>.norm1, .norm1b, .norm2, .norm2b (the latter two with a
  feed-forward only), attention: l<i>.mix.{q,k,v,o} and .mix.vmix (one number) where v_mix is set;
  latent attention: l<i>.mix.{dq,uq,dkv,uk,uv,o}, .mix.dq.norm [q_rank], .mix.dkv.norm [kv_rank];
  feed-forward: l<i>.mlp.{gate,up,down}.
"""
from dataclasses import dataclass, field

from .base import ConfigError, ModelConfig, get
from .nilivik import _freeze, _section, _thaw
from .specs import (GatedMLPSpec, LatentAttentionSpec, MaskedAttentionSpec, ModelSpec, RMSNormSpec, RotaryPairsSpec,
                    RotaryPartSpec, SandwichLayerSpec, UnitRMSNormSpec)


def _check_rot(m, where, limit, default_dims=None):
    rot = m.get("rot")
    if rot is None:
        return None
    rot = _section(m, "rot", where)
    dims = get(rot, "dims", int) if default_dims is None else get(rot, "dims", int, default_dims)
    if dims % 2 or not 0 <= dims <= limit:
        raise ConfigError(f"config.json: {where}.rot.dims {dims} must be even and at most {limit}")
    return {"dims": dims, "base": get(rot, "base", float, positive=True)}


def _check_mask(m, where):
    if m.get("mask") is None:
        return None
    return {"size": get(_section(m, "mask", where), "size", int, positive=True)}


def _check_mixer(kind, m, where):
    if kind == "attention":
        H = get(m, "heads", int, positive=True)
        G = get(m, "kv_heads", int, H, positive=True)
        if H % G:
            raise ConfigError(f"config.json: {where}: {H} heads are not a multiple of {G} key/value heads")
        dim = get(m, "dim", int, positive=True)
        out = {"heads": H, "kv_heads": G, "dim": dim, "vdim": get(m, "vdim", int, dim, positive=True),
               "scale": get(m, "scale", float), "v_mix": get(m, "v_mix", bool, False)}
        rot, mask = _check_rot(m, where, dim), _check_mask(m, where)
        if rot is not None:
            out["rot"] = rot
        if mask is not None:
            out["mask"] = mask
        return out
    if kind == "latent_attention":
        rd = get(m, "rot_dim", int, positive=True)
        out = {"heads": get(m, "heads", int, positive=True), "dim": get(m, "dim", int, positive=True), "rot_dim": rd,
               "vdim": get(m, "vdim", int, positive=True), "q_rank": get(m, "q_rank", int, positive=True),
               "kv_rank": get(m, "kv_rank", int, positive=True), "scale": get(m, "scale", float)}
        rot, mask = _check_rot(m, where, rd, default_dims=rd), _check_mask(m, where)
        if rot is None:
            raise ConfigError(f"config.json: {where}.rot (the base of the shared key part's rotation) is missing")
        out["rot"] = rot
        if mask is not None:
            out["mask"] = mask
        return out
    raise ConfigError(f"config.json: {where}.type {kind!r} is not implemented (attention, latent_attention)")


def _check_mlp(mlp, where):
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: {where}.mlp must be an object or null")
    if mlp.get("kind") != "dense":
        raise ConfigError(f"config.json: {where}.mlp kind {mlp.get('kind')!r} is not implemented (dense or null)")
    return {"kind": "dense", "ff": get(mlp, "ff", int, positive=True)}


@dataclass(frozen=True)
class VenidraConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    logit_scale: float
    logit_softcap: float                       # 0: logits are not capped
    layers: tuple = field(default=())          # the config's layer entries, checked, frozen

    architecture = "Venidra"

    @classmethod
    def from_dict(cls, d):
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        checked = []
        for i, lc in enumerate(layers):
            if not isinstance(lc, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            kind = lc.get("type")
            checked.append({"type": kind, "mixer": _check_mixer(kind, _section(lc, "mixer", f"layers[{i}]"), f"layers[{i}].mixer"),
                            "mlp": _check_mlp(lc.get("mlp"), f"layers[{i}]")})
        blend = [lc["mixer"] for lc in checked if lc["type"] == "attention" and lc["mixer"]["v_mix"]]
        if any(m["kv_heads"] * m["vdim"] != blend[0]["kv_heads"] * blend[0]["vdim"] or m["vdim"] != blend[0]["vdim"] for m in blend):
            raise ConfigError("config.json: layers that blend their values (v_mix) must have value heads of one shape")
        emb = d.get("embedding") or {}
        if not isinstance(emb, dict):
            raise ConfigError("config.json: 'embedding' must be an object")
        cap = get(d, "logit_softcap", float, 0.0)
        if cap < 0:
            raise ConfigError("config.json: 'logit_softcap' must not be negative")
        return cls(vocab=get(d, "vocab", int, positive=True), width=get(d, "width", int, positive=True),
                   norm_eps=get(_section(d, "norm", "the"), "eps", float, positive=True),
                   embedding_scale=get(emb, "scale", float, 1.0), logit_scale=get(d, "logit_scale", float, 1.0),
                   logit_softcap=cap, layers=tuple(_freeze(l) for l in checked))

    def layer_dicts(self):
        return [_thaw(l) for l in self.layers]

    def to_dict(self):
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale, "layers": self.layer_dicts()}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d

    def to_spec(self):
        W, eps = self.width, self.norm_eps
        norm = lambda: RMSNormSpec(W, eps, tensor="")
        layers, source_seen = [], False
        for i, lc in enumerate(self.layer_dicts()):
            m = lc["mixer"]
            mask, rot = m.get("mask"), m.get("rot")
            if lc["type"] == "attention":
                value_mix = None
                if m["v_mix"]:
                    value_mix, source_seen = ("blend" if source_seen else "source"), True
                mixer = MaskedAttentionSpec(
                    hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                    scale=m["scale"], chunk=mask["size"] if mask else None, qk_norm=UnitRMSNormSpec(m["dim"], eps),
                    position=RotaryPartSpec(rot["dims"], rot["base"]) if rot and rot["dims"] else None,
                    norm_after_rotation=True, value_mix=value_mix)
            else:
                mixer = LatentAttentionSpec(
                    hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_head_dim=m["vdim"],
                    q_rank=m["q_rank"], kv_rank=m["kv_rank"], scale=m["scale"], norm_eps=eps,
                    position=RotaryPairsSpec(rot["dims"], rot["base"]) if rot["dims"] else None,
                    window=mask["size"] if mask else None)
            ff = GatedMLPSpec(W, lc["mlp"]["ff"], "gelu_tanh", names=("gate", "up", "down")) if lc["mlp"] else None
            names = (("norm_in", "norm1"), ("mixer", "mix."), ("norm_mix_out", "norm1b")) + \
                ((("norm_post", "norm2"), ("feed_forward", "mlp."), ("norm_ff_out", "norm2b")) if ff else ())
            layers.append(SandwichLayerSpec(prefix=f"l{i}.", norm_in=norm(), mixer=mixer, norm_mix_out=norm(),
                                            norm_post=norm() if ff else None, feed_forward=ff,
                                            norm_ff_out=norm() if ff else None, names=names))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden_size=W, layers=tuple(layers),
                         schedule=ModelSpec.identity_schedule(len(layers)), final_norm=RMSNormSpec(W, eps, tensor=""),
                         tie_embeddings=True, max_positions=1 << 20, embed_name="embed", final_norm_prefix="final.norm",
                         head_name="head", embed_scale=self.embedding_scale, logit_cap=self.logit_softcap or None,
                         logit_scale=self.logit_scale,
                         # a blending weight may come with an attention layer that does not blend: nothing reads it
                         unused_tensors=tuple(f"l{i}.mix.vmix" for i, lc in enumerate(self.layer_dicts())
                                              if lc["type"] == "attention" and not lc["mixer"]["v_mix"]))
