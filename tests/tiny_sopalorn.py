"""Small Sopalorn configurations for the tests, and helpers to make their model folders.

They differ from each other in every size and option: one to four copies of the stream and the plain residual sum;
attention with one to six query heads a key/value head, keys and values of equal, different and odd widths, rotations of a
part of a head, a whole head and no channel, with and without blended frequencies, layers that read an earlier layer's keys
and values; lightning layers with decays from 0.3 to 1; parallel layers whose windows are one token, shorter than a page and
longer than the prompts, whose delta rules have one to three value heads a query/key head and one to five taps; dense
feed-forwards, experts with none, a few and many identity experts, with every expert chosen and with one, layers without a
feed-forward.
"""
from __future__ import annotations

import copy
import random

import numpy as np
import torch


def attention(heads, kv_heads, dim, vdim, scale, rot=None, kv_from=None, mlp=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        mixer["rot"] = rot
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def rotation(dims, base, scaling=None):
    out = {"dims": dims, "base": base}
    if scaling:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def lightning(heads, dim, vdim, decay, mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def parallel(left, right, mlp=None):
    """left: (heads, kv_heads, dim, vdim, scale, window); right: (heads, kv_heads, dim, vdim, conv)"""
    lh, lg, ld, lv, ls, window = left
    rh, rg, rd, rv, conv = right
    return {"type": "parallel", "mlp": mlp,
            "mixer": {"left": {"heads": lh, "kv_heads": lg, "dim": ld, "vdim": lv, "scale": ls, "mask": {"size": window}},
                      "right": {"heads": rh, "kv_heads": rg, "dim": rd, "vdim": rv, "conv": conv}}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts, identity, top, ff, scale):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}


def config(width, vocab, eps, streams, layers, embedding_scale=1.0, logit_scale=1.0):
    out = {"architecture": "Sopalorn", "width": width, "vocab": vocab, "norm": {"eps": eps}, "embedding": {"scale": embedding_scale},
           "logit_scale": logit_scale, "layers": layers}
    if streams is not None:
        out["streams"] = streams
    return out


CONFIGS = {
    # three copies; keys 24 and values 20 wide under a partial rotation with blended frequencies; a window shorter than a
    # page beside a delta rule of two value heads a key head and three taps; two identity experts among eight; a
    # lightning layer that only mixes; a last layer on the first layer's keys and values
    "A": config(96, 200, 1e-6, 3,
                [attention(6, 2, 24, 20, 0.25, rotation(16, 500.0, (4.0, 64, 8.0, 1.0)), mlp=dense(72, 1.5)),
                 parallel((4, 2, 16, 24, 0.3, 37), (4, 2, 24, 20, 3), mlp=moe(6, 2, 3, 40, 1.5)),
                 lightning(3, 16, 24, (0.5, 0.9, 0.99), mlp=None),
                 attention(6, 2, 24, 20, 0.25, rotation(16, 500.0, (4.0, 64, 8.0, 1.0)), kv_from=0, mlp=moe(5, 0, 2, 56, 1.0))],
                embedding_scale=0.7, logit_scale=0.3),
    # sizes the tensor-core attention kernels take (heads of 64, a whole-head rotation), four query heads a key/value
    # head, a window longer than a page, two copies, three identity experts
    "B": config(128, 333, 1e-5, 2,
                [lightning(2, 64, 64, (0.8, 0.97), mlp=moe(10, 3, 4, 64, 2.5)),
                 attention(8, 2, 64, 64, 0.11, rotation(64, 10000.0), mlp=dense(160, 3.0)),
                 parallel((4, 1, 64, 64, 0.12, 70), (2, 2, 64, 64, 4), mlp=dense(96, 7.0)),
                 attention(8, 2, 64, 64, 0.11, rotation(64, 10000.0), kv_from=1, mlp=moe(4, 1, 1, 32, 0.5))],
                embedding_scale=2.0, logit_scale=0.5),
    # multiples of nothing: a width that is no multiple of 8, odd widths, one copy of the stream (with weights), one tap,
    # a window of one token, no rotation, every expert chosen, more identity experts than choices
    "C": config(52, 101, 1e-5, 1,
                [parallel((3, 1, 10, 7, 0.4, 1), (3, 3, 10, 7, 1), mlp=moe(3, 0, 3, 20, 1.0)),
                 attention(3, 1, 10, 14, 0.4, None, mlp=dense(24, 0.5)),
                 lightning(5, 6, 9, (0.3, 0.6, 0.9, 1.0, 0.95), mlp=moe(2, 5, 2, 16, 3.0)),
                 attention(2, 2, 12, 6, 0.3, rotation(6, 100.0, (2.0, 16, 4.0, 0.5)), mlp=None)],
                embedding_scale=1.0, logit_scale=1.0),
    # no copies at all (the plain residual sum), three value heads a key head and five taps, a window longer than any
    # prompt of the tests, six query heads on one key/value head, two layers on one layer's keys
    "D": config(80, 160, 1e-5, None,
                [attention(6, 1, 32, 16, 0.2, rotation(8, 50.0, (16.0, 32, 2.0, 1.0)), mlp=dense(40, 2.0)),
                 parallel((2, 2, 96, 32, 0.1, 4000), (6, 2, 16, 24, 5), mlp=None),
                 attention(6, 1, 32, 16, 0.2, rotation(8, 50.0, (16.0, 32, 2.0, 1.0)), kv_from=0, mlp=moe(9, 1, 4, 16, 1.0)),
                 attention(6, 1, 32, 16, 0.2, rotation(8, 50.0, (16.0, 32, 2.0, 1.0)), kv_from=0, mlp=dense(24, 1.0))],
                embedding_scale=0.5, logit_scale=2.0),
    # four copies, a lightning layer of many small heads, an attention layer between two that borrow from different owners
    "E": config(64, 90, 1e-6, 4,
                [attention(4, 4, 16, 16, 0.3, rotation(16, 1000.0), mlp=None),
                 attention(2, 1, 8, 40, 0.5, rotation(4, 20.0), mlp=moe(4, 4, 2, 24, 2.0)),
                 attention(4, 4, 16, 16, 0.3, rotation(16, 1000.0), kv_from=0, mlp=dense(32, 4.0)),
                 lightning(8, 8, 8, (0.9,) * 8, mlp=dense(48, 2.5)),
                 attention(2, 1, 8, 40, 0.5, rotation(4, 20.0), kv_from=1, mlp=None)],
                embedding_scale=1.5, logit_scale=0.7),
}

# One parallel layer alone whose window decides: the attention's scores are scaled up until the softmax all but picks one key.
SHARP_WINDOW = config(64, 120, 1e-5, 2, [parallel((4, 2, 16, 16, 6.0, 23), (2, 1, 8, 8, 2))])
# One attention layer alone (every earlier key, a rotation), equally sharp: a far key decides.
SHARP_FAR = config(64, 120, 1e-5, 2, [attention(4, 2, 16, 16, 6.0, rotation(8, 100.0, (4.0, 64, 8.0, 1.0)))])
# Layers at the widths of a real model's layers: heads of 128 channels, experts of 512.
WIDE = config(1024, 1000, 1e-5, 2,
              [attention(8, 2, 128, 128, 128 ** -0.5, rotation(64, 10000.0, (16.0, 512, 24.0, 0.5)), mlp=moe(8, 2, 2, 512, 2.0)),
               parallel((8, 2, 128, 128, 128 ** -0.5, 100), (8, 4, 128, 128, 4), mlp=dense(2048, 7.0)),
               lightning(8, 128, 128, tuple(1.0 - 2.0 ** -(i + 2) for i in range(8)), mlp=dense(1024, 7.0)),
               attention(8, 2, 128, 128, 128 ** -0.5, rotation(64, 10000.0, (16.0, 512, 24.0, 0.5)), kv_from=0, mlp=None)],
              embedding_scale=1.0, logit_scale=0.25)
CONFIGS.update(wide=WIDE, sharp_window=SHARP_WINDOW, sharp_far=SHARP_FAR)


def random_config(rng):
    """A configuration drawn from ``rng`` (a random.Random): two to six layers of the three mixers with sizes that are and
    are not multiples of 8, 16 or 64, windows from one token to beyond the prompts, layers that borrow keys, experts with
    and without identity experts, layers without a feed-forward, one to four copies of the stream or none."""
    width = rng.choice([64, 96, 128, 160, 192, 256, 100, 72])
    layers, owners = [], []
    for i in range(rng.randrange(2, 7)):
        mlp = None
        if rng.random() > 0.15:
            if rng.random() < 0.4:
                mlp = dense(rng.choice([24, 64, 100, 136]), rng.choice([0.5, 2.0, 7.0]))
            else:
                experts, identity = rng.randrange(1, 13), rng.choice([0, 0, 1, 2, 4])
                mlp = moe(experts, identity, rng.randrange(1, min(4, experts + identity) + 1), rng.choice([16, 24, 40, 64, 96, 30]),
                          rng.choice([1.0, 2.0, 0.5, 2.5]))
        kind = rng.choice(["attention", "attention", "lightning", "parallel"])
        if kind == "attention":
            if owners and rng.random() < 0.35:
                j = rng.choice(owners)
                entry = copy.deepcopy(layers[j])
                entry["mixer"]["kv_from"] = j
                entry["mixer"]["heads"] = entry["mixer"]["kv_heads"] * rng.choice([1, 2, 3])
                entry["mlp"] = mlp
                layers.append(entry)
                continue
            kv = rng.choice([1, 1, 2, 3, 4])
            dim = rng.choice([8, 16, 24, 32, 40, 48, 64, 64, 80, 96, 128])
            rd = rng.choice([0, dim, dim // 2 - (dim // 2) % 2, 2 * rng.randrange(1, dim // 2 + 1)])
            scaling = rng.choice([None, (8.0, 2048, 24.0, 1.0), (4.0, 64, 8.0, 0.5), (40.0, 4096, 16.0, 2.0)])
            layers.append(attention(kv * rng.choice([1, 2, 3, 4, 6]), kv, dim, rng.choice([dim, dim, 8, 20, 64]),
                                    rng.choice([0.1, 0.2, 0.35, dim ** -0.5]),
                                    rotation(rd, rng.choice([100.0, 10000.0, 500000.0]), scaling) if rd else None, mlp=mlp))
            owners.append(i)
        elif kind == "lightning":
            heads = rng.randrange(1, 9)
            layers.append(lightning(heads, rng.choice([8, 16, 24, 40, 64, 128]), rng.choice([8, 16, 20, 32, 64, 96]),
                                    [rng.choice([0.3, 0.6, 0.9, 0.99, 0.999, 1.0]) for _ in range(heads)], mlp=mlp))
        else:
            kv, g = rng.choice([1, 2, 3]), rng.choice([1, 2, 3])
            dim = rng.choice([8, 16, 24, 32, 64, 96, 128])
            layers.append(parallel((kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([dim, dim, 16, 40]), rng.choice([0.1, 0.3, dim ** -0.5]),
                                    rng.choice([1, 2, 7, 31, 64, 65, 100, 5000])),
                                   (g * rng.choice([1, 2, 3]), g, rng.choice([8, 16, 24, 40, 64, 72, 128]), rng.choice([8, 16, 20, 32, 64, 96]),
                                    rng.randrange(1, 6)), mlp=mlp))
    return config(width, rng.randrange(100, 600), rng.choice([1e-5, 1e-6]), rng.choice([None, 1, 2, 2, 3, 4]), layers,
                  rng.choice([0.5, 1.0, 1.7]), rng.choice([0.25, 1.0, 0.6]))


def make_folder(tmp_path, which, seed=0, dtype=torch.float32, cfg=None):
    """Write a model folder with the package's random-weights mode; returns its path."""
    from dotllm_b200.config import config_from_dict
    from dotllm_b200.weights import write_random_model
    cfg_dict = copy.deepcopy(cfg or CONFIGS[which])
    folder = tmp_path / f"sopalorn_{which}_{seed}_{str(dtype).split('.')[-1]}"
    write_random_model(folder, config_from_dict(cfg_dict), seed, dtype=dtype)
    return folder


def read_folder(folder):
    """(config dict, weights as float64 arrays) as the plain implementation takes them."""
    import plain_llama
    cfg, weights = plain_llama.read_model_folder(folder)
    return cfg, {name: t.double().numpy() for name, t in weights.items()}


def plain_logits(cfg, w, tokens):
    """The plain implementation's logits as a float64 tensor [T, vocab]."""
    import plain_sopalorn
    return torch.from_numpy(np.ascontiguousarray(plain_sopalorn.forward(cfg, w, tokens)[0]))


def random_tokens(n, vocab, seed):
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


def rewrite(folder, change):
    """Read the folder's tensors, let ``change(tensors)`` edit the dict in place, write them back."""
    from dotllm_b200.weights.safetensors_io import SafetensorsFile, save_safetensors
    path = folder / "model.safetensors"
    with SafetensorsFile(path) as f:
        tensors = {n: f.tensor(n).clone() for n in f.names()}
    change(tensors)
    save_safetensors(path, tensors, metadata={"format": "pt"})
    return folder


def scale_tensors(folder, factors):
    """Multiply stored tensors by factors ({name: factor}); exact in the stored type for powers of two."""
    def change(tensors):
        for name, factor in factors.items():
            tensors[name] = (tensors[name].to(torch.float32) * factor).to(tensors[name].dtype)
    return rewrite(folder, change)
