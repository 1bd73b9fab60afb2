"""Small Komulorn configurations for the tests, and helpers to make their model folders.

They differ from each other in every size and option: widths, vocabularies, query heads per key/value head (1, 2, 3, 4,
20), key and value widths that are equal, smaller, larger, odd, and multiples of nothing, rotations of a part of a head,
a whole head and no channel at all, with and without the rescaled frequencies, layers that read an earlier layer's keys
and values (the layer before, and one further back), a layer without a feed-forward, experts with and without a shared
one, one choice, several, and every expert chosen, logits capped and not.
"""
from __future__ import annotations

import copy
import random

import torch


def rot(dims, base=10000.0, scaling=None):
    out = {"dims": dims, "base": base}
    if scaling:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def attention(heads, kv_heads, dim, vdim, scale, rotation=None, kv_from=None, mlp=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rotation:
        mixer["rot"] = rotation
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def moe(experts, top, ff, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def config(width, vocab, eps, layers, softcap=None):
    out = {"architecture": "Komulorn", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}
    if softcap:
        out["logit_softcap"] = softcap
    return out


CONFIGS = {
    # values wider than keys; three query heads a key/value head; a rotation of a part of the head with rescaled
    # frequencies; the second and the fourth layer read the first one's cache; a layer that only mixes
    "A": config(96, 200, 1e-6,
                [attention(6, 2, 24, 40, 0.3, rot(16, 500.0, (4.0, 64, 8.0, 2.0)), mlp=moe(5, 2, 56, shared=72)),
                 attention(6, 2, 24, 40, 0.25, rot(16, 500.0, (4.0, 64, 8.0, 2.0)), kv_from=0, mlp=moe(4, 1, 40)),
                 attention(4, 4, 16, 16, 0.2, rot(16, 10000.0), mlp=None),
                 attention(6, 2, 24, 40, 0.3, rot(16, 500.0, (4.0, 64, 8.0, 2.0)), kv_from=0, mlp=moe(3, 3, 24, shared=16))],
                softcap=12.0),
    # sizes the tensor-core attention kernels take (keys and values of 64, a whole-head rotation), four query heads a
    # key/value head, no cap on the logits
    "B": config(128, 333, 1e-5,
                [attention(8, 2, 64, 64, 0.11, rot(64, 10000.0, (8.0, 128, 16.0, 1.0)), mlp=moe(8, 2, 64, shared=64)),
                 attention(8, 2, 64, 64, 0.14, rot(64, 10000.0, (8.0, 128, 16.0, 1.0)), kv_from=0, mlp=moe(6, 3, 72))]),
    # multiples of nothing: a width that is no multiple of 8, odd value width, one key/value head, no rotation in the
    # second layer, every expert chosen in the first
    "C": config(52, 101, 1e-5,
                [attention(3, 1, 10, 7, 0.4, rot(6, 100.0), mlp=moe(3, 3, 20)),
                 attention(2, 2, 12, 18, 0.3, None, mlp=moe(7, 2, 16, shared=8)),
                 attention(2, 2, 12, 18, 0.35, None, kv_from=1, mlp=None)],
                softcap=5.0),
    # twenty query heads on one key/value head; values narrower than keys; keys of 32 with values of 96
    "D": config(80, 160, 1e-5,
                [attention(20, 1, 8, 4, 0.5, rot(8, 1000.0, (2.0, 32, 4.0, 0.5)), mlp=moe(2, 1, 24, shared=24)),
                 attention(4, 2, 32, 96, 0.2, rot(8, 50.0), mlp=moe(9, 4, 16))],
                softcap=30.0),
}

# One attention layer alone whose scores are scaled up until the softmax all but picks one key: a far key that the
# rotation, the page table or a shared cache gets wrong then changes whole rows of logits.
SHARP = config(64, 120, 1e-5, [attention(4, 2, 16, 24, 6.0, rot(8, 10000.0, (4.0, 96, 8.0, 1.0)))])
SHARP_SHARED = config(64, 120, 1e-5, [attention(4, 2, 16, 24, 6.0, rot(8, 10000.0, (4.0, 96, 8.0, 1.0))),
                                       attention(4, 2, 16, 24, 5.0, rot(8, 10000.0, (4.0, 96, 8.0, 1.0)), kv_from=0)])
# Two layers at the widths of a real model's layers (the second on the first one's cache): heads of 128 channels, half of
# them rotated, experts of 512.
WIDE = config(1024, 1000, 1e-5,
              [attention(8, 2, 128, 128, 128 ** -0.5, rot(64, 10000.0, (4.0, 2048, 32.0, 1.0)), mlp=moe(8, 2, 512, shared=512)),
               attention(8, 2, 128, 128, 0.1, rot(64, 10000.0, (4.0, 2048, 32.0, 1.0)), kv_from=0, mlp=moe(8, 2, 512, shared=512))],
              softcap=30.0)
CONFIGS["wide"] = WIDE
CONFIGS["sharp"] = SHARP
CONFIGS["sharp_shared"] = SHARP_SHARED


def random_config(rng):
    """A configuration drawn from ``rng`` (a random.Random): two to five layers; widths that are and are not multiples of 8
    or 64; one to four key/value heads with one to eight query heads each; key and value widths from 8 to 128, equal or
    not; a rotation of no channel, a part of the head or all of it, rescaled or not; layers that read an earlier layer's
    cache; two to 24 experts with one to four chosen, with and without a shared one; layers without a feed-forward."""
    width = rng.choice([64, 96, 128, 160, 192, 256, 320, 100, 72])
    layers, own = [], []
    for i in range(rng.randrange(2, 6)):
        mlp = None
        if rng.random() > 0.15:
            experts = rng.randrange(2, 25)
            mlp = moe(experts, rng.randrange(1, min(4, experts) + 1), rng.choice([16, 24, 40, 56, 64, 96, 100, 136, 30]),
                      shared=rng.choice([None, 16, 48, 128, 72]))
        if own and rng.random() < 0.35:
            j = rng.choice(own)
            mixer = copy.deepcopy(layers[j]["mixer"])
            mixer["scale"] = rng.choice([0.1, 0.2, 0.35])
            mixer["kv_from"] = j
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
            continue
        kv = rng.choice([1, 1, 2, 3, 4])
        heads = kv * rng.choice([1, 2, 3, 4, 6, 8])
        dim = rng.choice([8, 16, 24, 32, 40, 48, 64, 64, 80, 96, 128])
        vdim = rng.choice([dim, dim, 8, 16, 24, 40, 64, 80, 96, 128, 20])
        rd = rng.choice([0, dim, dim // 2 - (dim // 2) % 2, 2 * rng.randrange(1, dim // 2 + 1)])
        rotation = None
        if rd:
            scaling = rng.choice([None, (rng.choice([2.0, 4.0, 8.0]), rng.choice([32, 64, 512, 4096]), rng.choice([4.0, 16.0, 32.0]),
                                         rng.choice([0.5, 1.0, 2.0]))])
            rotation = rot(rd, rng.choice([100.0, 10000.0, 500000.0]), scaling)
        layers.append(attention(heads, kv, dim, vdim, rng.choice([0.1, 0.2, 0.35, dim ** -0.5]), rotation, mlp=mlp))
        own.append(i)
    return config(width, rng.randrange(100, 600), rng.choice([1e-5, 1e-6]), layers, softcap=rng.choice([None, 8.0, 30.0]))


def make_folder(tmp_path, which, seed=0, dtype=torch.float32, cfg=None):
    """Write a model folder with the package's random-weights mode; returns its path."""
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.weights import write_random_model
    cfg_dict = copy.deepcopy(cfg or CONFIGS[which])
    folder = tmp_path / f"komulorn_{which}_{seed}_{str(dtype).split('.')[-1]}"
    write_random_model(folder, config_from_dict(cfg_dict), seed, dtype=dtype)
    return folder


def read_folder(folder):
    """(config dict, weights) as the plain implementation takes them."""
    import plain_llama
    return plain_llama.read_model_folder(folder)


def random_tokens(n, vocab, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def rescale(folder, factors):
    """Multiply stored tensors by factors ({name: factor}) and write the folder's weights again (values stay exact
    in the stored type when the factor is a power of two)."""
    from dotllm_b200.weights.safetensors_io import SafetensorsFile, save_safetensors
    path = folder / "model.safetensors"
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    for name, factor in factors.items():
        tensors[name] = (tensors[name].to(torch.float32) * factor).to(tensors[name].dtype)
    save_safetensors(path, tensors, metadata={"format": "pt"})
    return folder


def sharp_folder(tmp_path, which, dtype=torch.float32, seed=0):
    """A folder of ``which`` ("sharp", "sharp_shared") whose query and key projections are scaled up (x16, biases x4) so
    that, with the configuration's large score scale, a query's softmax all but picks one key."""
    folder = make_folder(tmp_path, which, seed=seed, dtype=dtype)
    factors = {}
    for i, layer in enumerate(CONFIGS[which]["layers"]):
        factors[f"l{i}.mix.q"] = 16.0
        factors[f"l{i}.mix.q.b"] = 4.0
        if layer["mixer"].get("kv_from") is None:
            factors[f"l{i}.mix.k"] = 16.0
            factors[f"l{i}.mix.k.b"] = 4.0
    return rescale(folder, factors)
