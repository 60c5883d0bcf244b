"""Nevotar: a pre-norm decoder whose norms work in groups and whose layers mix in one of three ways: differential
attention (two softmax maps per head over the same values, a query temperature that grows with the position, no
rotation), HGRN2 (a linear recurrence whose forget gate also decides what is written), or two mixers side by side:
grouped-query attention with biases, a norm per q and k head, a rotation of the heads' first coordinates, head scores
mixed by a matrix before the softmax and a sliding window, beside a Mamba-2 state-space mixer. Each layer's feed-forward
is a mixture of experts with a sigmoid router whose weights stand on the experts' inputs, a clamped gate, and a shared
expert; or none. A layer may run on another layer's weights with a cache or state of its own. The head is the embedding.

config.json keys (every size, and every constant that differs between models of the design):
  architecture "Nevotar"; vocab, width; norm: {eps, groups};
  layers[i] = {type: "attention", mixer: {heads, kv_heads, dim, vdim, scale, diff, q_temp: {coef, every}}, mlp: ...}
            | {type: "hgrn2", mixer: {heads, dim, vdim}, mlp: ...}
            | {type: "parallel", mixer: {left: {heads, kv_heads, dim, vdim, scale, rot: {dims, base}, mask: {size}},
                                         right: {heads, vdim, state, groups, conv, norm_groups}, left_scale, right_scale}, mlp: ...}
     with mlp = {kind: "moe", expert: {ff, limit}, router: {experts, top}, shared: {ff, limit}} | null,
     and optionally weights_of: j (the layer has no tensors; it runs on layer j's; what its entry leaves out is layer j's).
  Left out: kv_heads = heads, vdim = dim, q_temp = none, rot = none, mask = none, shared = none, norm.groups = 1.
Tensors: embed, final.norm, and per layer with tensors l<i>.norm1, l<i>.norm2,
  attention: l<i>.mix.{q,k,v,o}, .mix.{q,k,v}.b, .mix.{lq1,lk1,lq2,lk2} [dim];
  hgrn2: l<i>.mix.{q,f,v,o}, .mix.f.b, .mix.lower [heads*dim], .mix.norm [vdim];
  parallel: l<i>.mix.left.{q,k,v,o}, .left.{q,k,v}.b, .left.{q,k}.norm [dim], .left.talk [heads, heads];
            l<i>.mix.right.{in,o}, .right.conv [channels, taps], .right.conv.b, .right.{dt_bias,A_log,D} [heads], .right.norm;
  moe: l<i>.mlp.e<k>.{gate,up,down}, .mlp.router, .mlp.shared.{gate,up,down}.
"""
from dataclasses import dataclass, field

from .base import ConfigError, ModelConfig, get
from .nilivik import _freeze, _section, _thaw
from .specs import (DiffAttentionSpec, GroupRMSNormSpec, LayerSpec, LowerBoundRecurrenceSpec, MaskedAttentionSpec, ModelSpec,
                    ParallelMixerSpec, RMSNormSpec, RotaryPartSpec, RoutedMLPSpec, ScheduleEntry, StateSpaceSpec)


def _heads(m, where):
    H = get(m, "heads", int, positive=True)
    G = get(m, "kv_heads", int, H, positive=True)
    if H % G:
        raise ConfigError(f"config.json: {where}: {H} heads are not a multiple of {G} key/value heads")
    dim = get(m, "dim", int, positive=True)
    return {"heads": H, "kv_heads": G, "dim": dim, "vdim": get(m, "vdim", int, dim, positive=True), "scale": get(m, "scale", float)}


def _check_mixer(kind, m, where):
    if kind == "attention":
        out = _heads(m, where)
        out["diff"] = get(m, "diff", float)
        if m.get("q_temp") is not None:
            qt = _section(m, "q_temp", where)
            out["q_temp"] = {"coef": get(qt, "coef", float), "every": get(qt, "every", int, positive=True)}
        return out
    if kind == "hgrn2":
        dim = get(m, "dim", int, positive=True)
        return {"heads": get(m, "heads", int, positive=True), "dim": dim, "vdim": get(m, "vdim", int, dim, positive=True)}
    if kind == "parallel":
        l, r = _section(m, "left", where), _section(m, "right", where)
        left = _heads(l, f"{where}.left")
        if l.get("rot") is not None:
            rot = _section(l, "rot", f"{where}.left")
            left["rot"] = {"dims": get(rot, "dims", int), "base": get(rot, "base", float, positive=True)}
            if left["rot"]["dims"] % 2 or not 0 <= left["rot"]["dims"] <= left["dim"]:
                raise ConfigError(f"config.json: {where}.left.rot.dims {left['rot']['dims']} must be even and at most dim")
        if l.get("mask") is not None:
            left["mask"] = {"size": get(_section(l, "mask", f"{where}.left"), "size", int, positive=True)}
        right = {"heads": get(r, "heads", int, positive=True), "vdim": get(r, "vdim", int, positive=True),
                 "state": get(r, "state", int, positive=True), "groups": get(r, "groups", int, 1, positive=True),
                 "conv": get(r, "conv", int, positive=True), "norm_groups": get(r, "norm_groups", int, 1, positive=True)}
        if right["heads"] % right["groups"] or (right["heads"] * right["vdim"]) % right["norm_groups"]:
            raise ConfigError(f"config.json: {where}.right: {right['heads']} heads of {right['vdim']} do not divide into "
                              f"{right['groups']} groups / {right['norm_groups']} norm groups")
        return {"left": left, "right": right, "left_scale": get(m, "left_scale", float, 1.0),
                "right_scale": get(m, "right_scale", float, 1.0)}
    raise ConfigError(f"config.json: {where}.type {kind!r} is not implemented (attention, hgrn2, parallel)")


def _check_mlp(mlp, where):
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"config.json: {where}.mlp must be an object or null")
    if mlp.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}.mlp kind {mlp.get('kind')!r} is not implemented (moe or null)")
    e, r = _section(mlp, "expert", f"{where}.mlp"), _section(mlp, "router", f"{where}.mlp")
    out = {"kind": "moe", "expert": {"ff": get(e, "ff", int, positive=True), "limit": get(e, "limit", float, positive=True)},
           "router": {"experts": get(r, "experts", int, positive=True), "top": get(r, "top", int, positive=True)}}
    if out["router"]["top"] > out["router"]["experts"]:
        raise ConfigError(f"config.json: {where}.mlp.router chooses {out['router']['top']} of {out['router']['experts']} experts")
    if mlp.get("shared") is not None:
        sh = _section(mlp, "shared", f"{where}.mlp")
        out["shared"] = {"ff": get(sh, "ff", int, positive=True), "limit": get(sh, "limit", float, positive=True)}
    return out


@dataclass(frozen=True)
class NevotarConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    layers: tuple = field(default=())          # the config's layer entries, checked, frozen

    architecture = "Nevotar"

    @classmethod
    def from_dict(cls, d):
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        checked = []
        for i, lc in enumerate(layers):
            if not isinstance(lc, dict):
                raise ConfigError(f"config.json: layers[{i}] must be an object")
            j = lc.get("weights_of")
            if isinstance(j, int) and not isinstance(j, bool) and 0 <= j < len(layers) and isinstance(layers[j], dict):
                lc = dict({k: v for k, v in layers[j].items() if k != "weights_of"}, **lc)   # left out: as layer j's
            kind = lc.get("type")
            entry = {"type": kind, "mixer": _check_mixer(kind, _section(lc, "mixer", f"layers[{i}]"), f"layers[{i}].mixer"),
                     "mlp": _check_mlp(lc.get("mlp"), f"layers[{i}]")}
            if lc.get("weights_of") is not None:
                entry["weights_of"] = get(lc, "weights_of", int)
            checked.append(entry)
        for i, lc in enumerate(checked):
            j = lc.get("weights_of")
            if j is None:
                continue
            if not 0 <= j < len(checked) or j == i or "weights_of" in checked[j]:
                raise ConfigError(f"config.json: layers[{i}].weights_of {j} must name another layer that has tensors of its own")
            if {k: v for k, v in lc.items() if k != "weights_of"} != checked[j]:
                raise ConfigError(f"config.json: layers[{i}] runs on the weights of layer {j} but is described differently")
        norm = _section(d, "norm", "the")
        width, groups = get(d, "width", int, positive=True), get(norm, "groups", int, 1, positive=True)
        if width % groups:
            raise ConfigError(f"config.json: norm.groups {groups} does not divide the width {width}")
        return cls(vocab=get(d, "vocab", int, positive=True), width=width, norm_eps=get(norm, "eps", float, positive=True),
                   norm_groups=groups, layers=tuple(_freeze(l) for l in checked))

    def layer_dicts(self):
        return [_thaw(l) for l in self.layers]

    def to_dict(self):
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps, "groups": self.norm_groups}, "layers": self.layer_dicts()}

    def owners(self):
        """Per layer the layer whose tensors it runs on (itself unless it says weights_of)."""
        return [lc.get("weights_of", i) for i, lc in enumerate(self.layer_dicts())]

    def _mixer_spec(self, kind, m):
        W, eps = self.width, self.norm_eps
        if kind == "attention":
            qt = m.get("q_temp")
            return DiffAttentionSpec(hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                     v_head_dim=m["vdim"], scale=m["scale"], diff=m["diff"], norm_eps=eps,
                                     q_temp=(qt["coef"], qt["every"]) if qt else None)
        if kind == "hgrn2":
            return LowerBoundRecurrenceSpec(hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"], norm_eps=eps)
        l, r = m["left"], m["right"]
        rot, mask = l.get("rot"), l.get("mask")
        left = MaskedAttentionSpec(hidden_size=W, num_heads=l["heads"], num_kv_heads=l["kv_heads"], head_dim=l["dim"],
                                   v_head_dim=l["vdim"], scale=l["scale"], window=mask["size"] if mask else None,
                                   qk_norm=RMSNormSpec(l["dim"], eps),
                                   position=RotaryPartSpec(rot["dims"], rot["base"]) if rot and rot["dims"] else None,
                                   bias=True, talk=True)
        right = StateSpaceSpec(hidden_size=W, num_heads=r["heads"], v_head_dim=r["vdim"], state_dim=r["state"], groups=r["groups"],
                               conv_taps=r["conv"], norm_groups=r["norm_groups"], norm_eps=eps)
        return ParallelMixerSpec(hidden_size=W, branches=(("left.", left, m["left_scale"]), ("right.", right, m["right_scale"])))

    def to_spec(self):
        W, eps, groups = self.width, self.norm_eps, self.norm_groups
        dicts, owners = self.layer_dicts(), self.owners()
        own = sorted(set(owners))                  # layers with tensors of their own, in order
        index = {i: k for k, i in enumerate(own)}
        norm = GroupRMSNormSpec(W, eps, groups)
        layers = []
        for i in own:
            lc, mlp = dicts[i], dicts[i]["mlp"]
            ff = None
            if mlp is not None:
                sh = mlp.get("shared")
                ff = RoutedMLPSpec(hidden_size=W, expert_ff=mlp["expert"]["ff"], num_experts=mlp["router"]["experts"],
                                   top=mlp["router"]["top"], shared_ff=sh["ff"] if sh else None, activation="clamped",
                                   correction=False, renorm=False, weight_on_input=True, shared_gate=False,
                                   limit=mlp["expert"]["limit"], shared_limit=sh["limit"] if sh else None)
            names = (("norm_in", "norm1"), ("mixer", "mix.")) + ((("norm_post", "norm2"), ("feed_forward", "mlp.")) if ff else ())
            layers.append(LayerSpec(prefix=f"l{i}.", norm_in=norm, mixer=self._mixer_spec(lc["type"], lc["mixer"]),
                                    norm_post=norm if ff else None, feed_forward=ff, names=names))
        schedule = tuple(ScheduleEntry(layer=index[o], cache=k, writes=True) for k, o in enumerate(owners))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden_size=W, layers=tuple(layers),
                         schedule=schedule, final_norm=norm, tie_embeddings=True, max_positions=1 << 20, embed_name="embed",
                         final_norm_prefix="final.norm")
