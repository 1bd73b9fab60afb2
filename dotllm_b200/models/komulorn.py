"""The Komulorn decoder as a model description.

Token embedding; pre-norm layers (plain RMSNorm gains) of softmax attention and a mixture of experts (or no
feed-forward); a final norm, a head of its own and a cap c tanh(logits / c) on the logits.

Attention: grouped key/value heads, key and value channels of different widths, biases on q, k and v, a rotation of
the first ``rot.dims`` channels of every head in the half-split pairing with frequencies blended per index over a ramp
("yarn") and cos / sin grown by 0.1 ln(factor) + 1, the configuration's own score scale, causal softmax, and a gate
sigmoid(g_h . x) on each head's output before the output projection.  A layer with ``kv_from`` has no key and value
projections: it attends with its own queries over the cache of the layer it names (the schedule's ``cache_of``).

Feed-forward: a router's sigmoid scores choose ``top`` experts (ties to the lower index); a chosen expert's score, not
renormalised, multiplies the expert's INPUT; an expert is down(relu(up x)^2) without biases; a shared expert of the
same form runs for every token, times sigmoid(sg . x).

Tensor names: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.q|k|v`` (+ ``.b``), ``l<i>.mix.g|o``, ``l<i>.mlp.e<j>.up|down``,
``l<i>.mlp.router``, ``l<i>.mlp.shared.up|down|sg``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.komulorn import KomulornConfig
from ..config.registry import register_architecture
from ..config.spec import LayerPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

EXPERT_ACTIVATION = "relu2"        # the experts' activation is the square of relu: fixed by the design


def _norm(cfg, name):
    return PartSpec("rmsnorm", {"eps": cfg.eps, "tensor": ""}, name)


def _mixer(cfg, m, prefix):
    position = None
    if m.rot_dims:
        s = m.rot_scaling
        scaling = None if s is None else {"rope_type": "yarn", "factor": s.factor, "original_max_position_embeddings": s.original,
                                          "fast_turns": s.fast, "slow_turns": s.slow}
        position = {"kind": "rotary", "params": {"rotary_dim": m.rot_dims, "theta": m.rot_base, "head_dim": m.dim,
                                                 "max_positions": cfg.max_positions, "scaling": scaling}}
    return PartSpec("attention",
                    {"n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim, "scale": m.scale,
                     "window": None, "position": position, "bias": True, "gate": "head_sigmoid", "own_kv": m.kv_from is None,
                     "tensors": {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g", "q_bias": "q.b", "k_bias": "k.b",
                                 "v_bias": "v.b"}}, prefix)


def _feed_forward(mlp, prefix):
    shared = {"intermediate_size": mlp.shared_ff, "gate": True} if mlp.shared_ff else None
    return PartSpec("routed_experts",
                    {"n_experts": mlp.experts, "top": mlp.top, "intermediate_size": mlp.ff, "activation": EXPERT_ACTIVATION,
                     "router_bias": False, "scoring": "sigmoid", "weight_on": "input", "shared": shared,
                     "tensors": {"expert": "e{e}.{m}", "router": "router", "shared": "shared.{m}", "shared_gate": "shared.sg"}},
                    prefix)


def build_komulorn_spec(cfg: KomulornConfig) -> ModelSpec:
    layers, unused = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = [LayerPart("mixer_norm", "norm", _norm(cfg, p + "norm1")),
                 LayerPart("mixer", "mixer", _mixer(cfg, layer.mixer, p + "mix."))]
        if layer.mlp is not None:
            parts += [LayerPart("feed_forward_norm", "norm", _norm(cfg, p + "norm2")),
                      LayerPart("feed_forward", "feed_forward", _feed_forward(layer.mlp, p + "mlp."))]
        else:                                                   # a checkpoint may still carry the absent sublayer's norm
            unused.append(p + "norm2")
        layers.append(LayerSpec("pre_norm", tuple(parts)))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "tensor": "embed", "init_std": 0.5}, ""),
        layers=tuple(layers),
        # one execution per layer; a layer that reads another's keys and values shares that execution's cache
        schedule=tuple(ScheduleEntry(i, layer.mixer.kv_from) for i, layer in enumerate(cfg.layers)),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "softcap": cfg.logit_softcap, "tensor": ""}, "head"),
        stop_token_ids=tuple(cfg.eos_token_id),
        bos_token_id=cfg.bos_token_id,
        optional_weights=tuple(unused))


register_architecture("Komulorn", KomulornConfig, build_komulorn_spec, model_types=("komulorn",))
