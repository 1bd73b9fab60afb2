"""Small Kubedra configurations for the tests, and helpers to make their model folders.

They differ from each other in every size and option: widths, heads, key / value sizes that are and are not
multiples of 8 or 32, latent ranks that the tensor-core attention kernels take (64, 128) and do not (40, 24),
windows shorter and longer than a cache page, a layer without a feed-forward, experts with and without a
shared one, top 1 and top 3, a repeated run at the start, in the middle and none, decay ranks that only the
tensors give.
"""
from __future__ import annotations

import copy
import json
import random

import torch


def gla(heads, dim, vdim, tau, mlp, rank=None):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}
    if rank is not None:
        mixer["decay_rank"] = rank
    return {"type": "gla", "mixer": mixer, "mlp": mlp}


def latent(heads, dim, vdim, q_rank, kv_rank, window=None, scale=None, mlp=None):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank}
    if window is not None:
        mixer["mask"] = {"size": window}
    if scale is not None:
        mixer["scale"] = scale
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, shared=None):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def config(width, vocab, positions, eps, layers, loop=None):
    out = {"architecture": "Kubedra", "width": width, "vocab": vocab, "max_positions": positions, "norm": {"eps": eps},
           "layers": layers}
    if loop:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


CONFIGS = {
    # a run of two layers at the start that repeats; a layer that only mixes; windows on both sides of a page
    "P": config(96, 200, 400, 1e-6,
                [latent(3, 24, 40, 48, 64, window=70, scale=0.2, mlp=dense(136)),
                 gla(3, 20, 24, 8.0, moe(5, 2, 56, 1.5, shared=(72, 2.5)), rank=6),
                 gla(2, 16, 48, 3.0, None, rank=4),
                 latent(2, 16, 24, 32, 40, window=33, mlp=moe(4, 1, 40, 3.0))],
                loop=(0, 2, 2)),
    # one layer in the middle that runs three times; a latent the tcgen05 kernel takes; one head; no window
    "Q": config(128, 333, 700, 1e-5,
                [gla(1, 64, 64, 4.0, dense(200), rank=16),
                 latent(4, 32, 32, 64, 128, window=130, mlp=moe(6, 3, 64, 2.0, shared=(32, 1.0))),
                 latent(5, 8, 16, 24, 24, mlp=dense(100))],
                loop=(1, 2, 3)),
    # nothing repeats; sizes that are multiples of nothing
    "R": config(72, 150, 300, 1e-5,
                [gla(3, 10, 14, 16.0, moe(3, 3, 20, 2.0), rank=3),
                 latent(3, 12, 10, 20, 36, window=5, mlp=dense(50))]),
    # everything repeats (the run is the whole model and ends in a layer without a feed-forward); a width that is no
    # multiple of 8; more heads than the decode attention kernel takes on one shared head; an odd latent; a window of one
    # token and one of exactly a page; a decay of rank 1; every expert but five chosen
    "S": config(52, 101, 300, 1e-5,
                [latent(20, 8, 8, 16, 64, window=64, mlp=moe(2, 2, 24, 1.0)),
                 gla(5, 6, 3, 2.0, dense(30), rank=2),
                 gla(1, 33, 65, 1.5, moe(9, 4, 16, 0.5, shared=(8, 4.0)), rank=1),
                 latent(1, 4, 4, 4, 37, window=1, mlp=None)],
                loop=(0, 4, 2)),
    # latents of 96 and 32: the widths that the mma.sync prefill attention and the decode kernel take besides 64 and 128
    "T": config(80, 160, 400, 1e-5,
                [latent(4, 16, 24, 40, 96, window=100, mlp=dense(64)),
                 latent(2, 24, 16, 24, 32, mlp=moe(4, 2, 32, 2.0, shared=(16, 2.0))),
                 gla(2, 32, 32, 8.0, None, rank=8)]),
}

# One mixer alone, for tests that isolate a mechanism.  The latent layer's scores are scaled up until the softmax
# all but picks one key, so that a window that is one token off changes whole rows of logits.
LATENT_ONLY = config(64, 120, 400, 1e-5, [latent(2, 16, 16, 32, 64, window=37, scale=6.0)])
GLA_ONLY = config(64, 120, 700, 1e-5, [gla(2, 24, 16, 64.0, None, rank=5)])
CONFIGS["latent_only"] = LATENT_ONLY
CONFIGS["gla_only"] = GLA_ONLY


def make_folder(tmp_path, which, seed=0, dtype=torch.float32, cfg=None):
    """Write a model folder with the package's random-weights mode; returns its path."""
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.weights import write_random_model
    cfg_dict = copy.deepcopy(cfg or CONFIGS[which])
    folder = tmp_path / f"kubedra_{which}_{seed}_{str(dtype).split('.')[-1]}"
    write_random_model(folder, config_from_dict(cfg_dict), seed, dtype=dtype)
    return folder


def read_folder(folder):
    """(config dict, weights) as the plain implementation takes them."""
    import plain_llama
    return plain_llama.read_model_folder(folder)


def random_tokens(n, vocab, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]
