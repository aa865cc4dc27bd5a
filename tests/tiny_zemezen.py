"""Small Zemezen configurations for the tests, and helpers to make their model folders.

They differ from each other in every size and option: widths and vocabularies; delta-rule layers with one to three value
heads a query/key head, key and value widths that are equal, different, odd, convolutions of one to five taps; latent
attention with latents smaller and larger than the heads; attention with one to six query heads a key/value head, rotations
of a part of a head, a whole head and no channel, windows shorter than a page, longer than the prompts and of one token,
no kept first tokens, a few, more than a page and more than the window; dense feed-forwards, experts with and without
groups (groups of one expert, every group kept, every expert chosen), layers without a feed-forward; layers that run with
another layer's weights (the first, a middle one, twice).
"""
from __future__ import annotations

import copy
import random

import torch


def delta(heads, kv_heads, dim, vdim, conv, mlp=None, ranks=None, weights_of=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}
    if ranks:
        mixer["ranks"] = list(ranks)
    return _layer("channel_delta", mixer, mlp, weights_of)


def latent(heads, dim, vdim, kv_rank, scale, mlp=None, weights_of=None):
    return _layer("latent_attention", {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}, mlp, weights_of)


def attention(heads, kv_heads, dim, scale, window, keep_first, rot_dims, rot_base=10000.0, mlp=None, weights_of=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
             "mask": {"size": window, "keep_first": keep_first}, "rot": {"dims": rot_dims, "base": rot_base}}
    return _layer("attention", mixer, mlp, weights_of)


def _layer(kind, mixer, mlp, weights_of):
    out = {"type": kind, "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None):
    router = {"experts": experts, "top": top}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def config(width, vocab, eps, layers):
    return {"architecture": "Zemezen", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


def again(layers, j, **changes):
    """Layer j's entry once more, running with layer j's weights."""
    out = copy.deepcopy(layers[j])
    out["weights_of"] = j
    return out


def _with_repeats(layers, repeats):
    for j in repeats:
        layers.append(again(layers, j))
    return layers


CONFIGS = {
    # two value heads a query/key head, three taps; a latent larger than the heads; a window shorter than a page with three
    # kept tokens and a rotation of a part of the head; experts in three groups of which two stay; a layer that only
    # mixes; the delta layer and the attention layer run again at the end with their weights
    "A": config(96, 200, 1e-6, _with_repeats(
        [delta(4, 2, 24, 20, 3, mlp=dense(72)),
         latent(3, 16, 24, 40, 0.3, mlp=moe(6, 2, 40, groups=(3, 2))),
         attention(6, 2, 24, 0.25, 37, 3, 16, 500.0, mlp=moe(5, 3, 56)),
         attention(4, 4, 16, 0.3, 50, 0, 16, mlp=None)], [0, 2])),
    # sizes the tensor-core attention kernels take (heads and latents of 64, a whole-head rotation), four query heads a
    # key/value head, a window longer than a page, more kept tokens than a page holds
    "B": config(128, 333, 1e-5,
                [attention(8, 2, 64, 0.11, 70, 5, 64, mlp=dense(160)),
                 delta(2, 2, 64, 64, 4, mlp=moe(10, 4, 64, groups=(5, 3))),
                 latent(4, 32, 48, 64, 0.17, mlp=dense(96)),
                 attention(4, 1, 128, 0.09, 130, 70, 64, 1000000.0, mlp=moe(4, 1, 32, groups=(4, 4)))]),
    # multiples of nothing: a width that is no multiple of 8, odd key and value widths, one tap, a window of one token,
    # no rotation, every expert chosen, groups of one expert, a layer run three times
    "C": config(52, 101, 1e-5, _with_repeats(
        [delta(3, 3, 10, 7, 1, mlp=moe(3, 3, 20)),
         attention(3, 1, 10, 0.4, 1, 2, 6, 100.0, mlp=dense(24)),
         latent(2, 12, 5, 24, 0.35, mlp=moe(6, 2, 16, groups=(6, 3))),
         attention(2, 2, 12, 0.3, 9, 0, 0, mlp=None)], [1, 1])),
    # three value heads a query/key head and five taps; a window longer than any prompt of the tests; kept tokens beyond
    # the window's size; six query heads on one key/value head
    "D": config(80, 160, 1e-5,
                [delta(6, 2, 16, 24, 5, mlp=None, ranks=(4, 9)),
                 attention(6, 1, 32, 0.2, 4000, 2, 8, 50.0, mlp=dense(40)),
                 attention(2, 2, 96, 0.1, 6, 11, 96, mlp=moe(9, 4, 16))]),
}

# One attention layer alone whose scores are scaled up until the softmax all but picks one key: a key just inside or just
# outside the window, a kept first token or the one behind it then changes whole rows of logits.
SHARP = config(64, 120, 1e-5, [attention(4, 2, 16, 6.0, 23, 3, 8)])
# Two layers at the widths of a real model's layers: heads of 128 channels, latents of 128, experts of 512.
WIDE = config(1024, 1000, 1e-5,
              [attention(8, 2, 128, 128 ** -0.5, 100, 4, 64, mlp=moe(8, 2, 512, groups=(4, 2))),
               delta(8, 4, 128, 128, 4, mlp=dense(2048)),
               latent(8, 64, 64, 128, 0.125, mlp=dense(1024))])
CONFIGS["wide"] = WIDE
CONFIGS["sharp"] = SHARP


def random_config(rng):
    """A configuration drawn from ``rng`` (a random.Random): two to six layers of the three mixers with sizes that are and
    are not multiples of 8, 16 or 64, windows from one token to beyond the prompts, kept tokens from none to beyond a page,
    experts with and without groups, layers without a feed-forward and layers that run with an earlier layer's weights."""
    width = rng.choice([64, 96, 128, 160, 192, 256, 100, 72])
    layers, own = [], []
    for i in range(rng.randrange(2, 7)):
        if own and rng.random() < 0.25:
            layers.append(again(layers, rng.choice(own)))
            continue
        mlp = None
        if rng.random() > 0.15:
            if rng.random() < 0.4:
                mlp = dense(rng.choice([24, 64, 100, 136]))
            else:
                count = rng.choice([1, 2, 3, 4])
                per = rng.randrange(1, 5)
                keep = rng.randrange(1, count + 1)
                top = rng.randrange(1, min(4, keep * per) + 1)
                mlp = moe(count * per, top, rng.choice([16, 24, 40, 64, 96, 30]), groups=(count, keep) if rng.random() < 0.7 else None)
        kind = rng.choice(["channel_delta", "latent_attention", "attention"])
        if kind == "channel_delta":
            kv = rng.choice([1, 2, 3])
            layers.append(delta(kv * rng.choice([1, 2, 3]), kv, rng.choice([8, 16, 24, 40, 64, 72, 128]),
                                rng.choice([8, 16, 20, 32, 64, 96]), rng.randrange(1, 6), mlp=mlp))
        elif kind == "latent_attention":
            layers.append(latent(rng.randrange(1, 9), rng.choice([8, 16, 24, 40, 64]), rng.choice([8, 16, 20, 48, 64]),
                                 rng.choice([16, 32, 40, 64, 96, 128]), rng.choice([0.1, 0.2, 0.35]), mlp=mlp))
        else:
            kv = rng.choice([1, 1, 2, 3, 4])
            dim = rng.choice([8, 16, 24, 32, 40, 48, 64, 64, 80, 96, 128])
            rd = rng.choice([0, dim, dim // 2 - (dim // 2) % 2, 2 * rng.randrange(1, dim // 2 + 1)])
            layers.append(attention(kv * rng.choice([1, 2, 3, 4, 6]), kv, dim, rng.choice([0.1, 0.2, 0.35, dim ** -0.5]),
                                    rng.choice([1, 2, 7, 31, 64, 65, 100, 5000]), rng.choice([0, 0, 1, 4, 63, 64, 70]), rd,
                                    rng.choice([100.0, 10000.0, 500000.0]), mlp=mlp))
        own.append(i)
    return config(width, rng.randrange(100, 600), rng.choice([1e-5, 1e-6]), layers)


def make_folder(tmp_path, which, seed=0, dtype=torch.float32, cfg=None):
    """Write a model folder with the package's random-weights mode; returns its path."""
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.weights import write_random_model
    cfg_dict = copy.deepcopy(cfg or CONFIGS[which])
    folder = tmp_path / f"zemezen_{which}_{seed}_{str(dtype).split('.')[-1]}"
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


def sharp_folder(tmp_path, dtype=torch.float32, seed=0, sink=None, gains=2.0):
    """A folder of the sharp configuration whose query and key norms' gains are scaled up (the norms undo any scale on
    the projections), so that with the configuration's large score scale a query's softmax all but picks one key;
    ``sink`` sets every head's sink.  With ``gains`` 0.25 the scores stay of order one instead, and a sink of that order
    takes a visible share of every row's softmax."""
    folder = make_folder(tmp_path / f"gains{gains}_sink{sink}", "sharp", seed=seed, dtype=dtype)
    rescale(folder, {"l0.mix.q.norm": gains, "l0.mix.k.norm": gains, "l0.mix.o": 16.0})       # and the mixer outweighs the embedding
    if sink is not None:
        from dotllm_b200.weights.safetensors_io import SafetensorsFile, save_safetensors
        path = folder / "model.safetensors"
        with SafetensorsFile(path) as f:
            tensors = {n: f.tensor(n).clone() for n in f.names()}
        tensors["l0.mix.sink"] = torch.full_like(tensors["l0.mix.sink"], sink)
        save_safetensors(path, tensors, metadata={"format": "pt"})
    return folder
