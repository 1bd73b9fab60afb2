"""The Kubedra decoder as a model description.

Token embedding plus learned absolute positions; layers with a norm before and behind each sublayer whose
gains are stored around zero; per layer one of two mixers - gated linear attention (a recurrent state) or
latent attention without positions under a sliding window (a paged cache of latents) - and a dense
gelu-gated feed-forward, a routed one with an optional shared expert, or none; a run of layers that repeats
with shared weights, every pass with a cache of its own and, from the second pass on, the embedding output
taken in again before its first layer; a final norm and a head that is the embedding table.
Tensor names: ``embed``, ``pos``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

from ..config.kubedra import KubedraConfig
from ..config.registry import register_architecture
from ..config.spec import LayerPart, LayerSpec, ModelSpec, PartSpec, ScheduleEntry

EXPERT_ALPHA = 1.702            # the experts' gate is g sigmoid(1.702 g): fixed by the design


def _norm(cfg, name):
    return PartSpec("rmsnorm", {"eps": cfg.eps, "offset": 1.0, "tensor": ""}, name)


def _mixer(cfg, layer, prefix):
    m = layer.mixer
    if layer.type == "gla":
        params = {"n_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "tau": m.tau, "eps": cfg.eps,
                  "tensors": {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm",
                              "decay_in": "a1", "decay_out": "a2", "decay_bias": "a2.b"}}
        if m.decay_rank is not None:
            params["decay_rank"] = m.decay_rank
        return PartSpec("gated_linear_attention", params, prefix)
    return PartSpec("latent_attention",
                    {"n_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank,
                     "eps": cfg.eps, "scale": m.scale, "window": m.window,
                     "tensors": {"q_down": "dq", "q_norm": "dq.norm", "q_up": "uq", "kv_down": "dkv",
                                 "kv_norm": "dkv.norm", "k_up": "uk", "v_up": "uv", "out": "o"}}, prefix)


def _feed_forward(mlp, prefix):
    if mlp.kind == "dense":
        return PartSpec("gated_mlp", {"intermediate_size": mlp.ff, "activation": "gelu_tanh",
                                      "tensors": ("gate", "up", "down")}, prefix)
    shared = {"intermediate_size": mlp.shared_ff, "limit": mlp.shared_limit} if mlp.shared_ff else None
    return PartSpec("routed_experts",
                    {"n_experts": mlp.experts, "top": mlp.top, "intermediate_size": mlp.ff,
                     "activation": "clamped_sigmoid", "limit": mlp.limit, "alpha": EXPERT_ALPHA, "router_bias": True,
                     "shared": shared,
                     "tensors": {"expert": "e{e}.{m}", "router": "router", "router_bias": "router.b",
                                 "shared": "shared.{m}"}}, prefix)


def build_kubedra_spec(cfg: KubedraConfig) -> ModelSpec:
    layers, unused = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        if layer.mlp is None:                                  # a checkpoint may still carry the absent sublayer's norms
            unused += [p + "norm2", p + "norm2b"]
        parts = [LayerPart("mixer_norm", "norm", _norm(cfg, p + "norm1")),
                 LayerPart("mixer", "mixer", _mixer(cfg, layer, p + "mix.")),
                 LayerPart("mixer_post_norm", "norm", _norm(cfg, p + "norm1b"))]
        if layer.mlp is not None:
            parts += [LayerPart("feed_forward_norm", "norm", _norm(cfg, p + "norm2")),
                      LayerPart("feed_forward", "feed_forward", _feed_forward(layer.mlp, p + "mlp.")),
                      LayerPart("feed_forward_post_norm", "norm", _norm(cfg, p + "norm2b"))]
        layers.append(LayerSpec("sandwich_norm", tuple(parts)))
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        max_positions=cfg.max_positions,
        embedding=PartSpec("token_position_embedding",
                           {"vocab_size": cfg.vocab, "max_positions": cfg.max_positions,
                            "token_tensor": "embed", "position_tensor": "pos", "init_std": 0.5}, ""),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, None, again) for i, again in cfg.layer_runs()),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab}, "head."),
        stop_token_ids=tuple(cfg.eos_token_id),
        bos_token_id=cfg.bos_token_id,
        shared_weights=(("head.weight", "embed"),),
        optional_weights=tuple(unused))


register_architecture("Kubedra", KubedraConfig, build_kubedra_spec, model_types=("kubedra",))
