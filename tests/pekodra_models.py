"""Tiny Pekodra configurations for the tests: every size differs between them and between their layers, and the
values that make two mechanisms coincide (keys as wide as values, one kv head, a rotation over the whole head, one
expert a row, a single walk of the loop) appear in one layer and not in the next."""


def attention(heads, kv_heads, dim, vdim, window, rot, scale):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if rot is not None:
        dims, base, scaling = rot
        mixer["rot"] = {"dims": dims, "base": base}
        if scaling is not None:
            factor, original, fast, slow = scaling
            mixer["rot"]["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return mixer


def layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


TINY_PEKODRA = {
    # the loop in the middle and walked twice; windows of 21 and 5 (shorter than a page) and a layer that sees all;
    # rotation over part of the head with stretched frequencies, over the whole head without, and none
    "a": {"architecture": "Pekodra", "width": 48, "vocab": 131, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.5},
          "logit_scale": 0.5, "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [layer(attention(4, 2, 16, 24, 21, (8, 1000.0, (3.0, 64, 8.0, 1.0)), 0.2), dense(72)),
                     layer(attention(3, 3, 24, 8, 5, (24, 50.0, None), 0.3), moe(5, 2, 24, 40)),
                     layer(attention(2, 1, 32, 32, None, None, 0.15), dense(40)),
                     layer(attention(6, 2, 8, 16, 40, (4, 10000.0, (8.0, 32, 4.0, 0.5)), 0.35), moe(4, 1, 32, None))]},
    # the loop from the first layer to the last, three walks, one layer without a feed-forward; every expert taken
    "b": {"architecture": "Pekodra", "width": 64, "vocab": 256, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
          "logit_scale": 2.0, "loop": {"start": 0, "stop": 2, "times": 3},
          "layers": [layer(attention(2, 1, 32, 16, 33, (32, 100.0, (2.0, 16, 2.0, 1.0)), 0.2), moe(3, 3, 32, 64)),
                     layer(attention(4, 4, 16, 16, 16, (16, 7.0, None), 0.25), None)]},
    # no loop at all; a window wider than any prompt of the tests; widths that are no multiple of four or eight
    "c": {"architecture": "Pekodra", "width": 42, "vocab": 77, "norm": {"eps": 1e-4}, "embedding": {"scale": 0.7},
          "logit_scale": 1.0,
          "layers": [layer(attention(1, 1, 20, 10, 1000, (10, 30.0, (4.0, 40, 32.0, 1.0)), 0.2), moe(7, 2, 12, 9)),
                     layer(attention(3, 1, 6, 12, 9, (6, 3.0, None), 0.5), dense(30))]},
    # a single walk of a loop that is the last layer alone; a window of one position
    "d": {"architecture": "Pekodra", "width": 32, "vocab": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0},
          "logit_scale": 0.125, "loop": {"start": 1, "stop": 2, "times": 1},
          "layers": [layer(attention(2, 2, 8, 8, 1, (8, 20.0, None), 0.4), dense(16)),
                     layer(attention(4, 1, 16, 8, 17, (12, 500.0, (16.0, 8, 1.0, 0.25)), 0.2), moe(9, 4, 8, 16))]},
    # head sizes and prompt lengths that send prompt portions to the tensor-core attention: a window, and all keys
    "e": {"architecture": "Pekodra", "width": 64, "vocab": 90, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5},
          "logit_scale": 0.5, "loop": {"start": 0, "stop": 1, "times": 2},
          "layers": [layer(attention(2, 1, 64, 64, 100, (32, 10000.0, (4.0, 128, 16.0, 1.0)), 0.125), dense(48)),
                     layer(attention(4, 2, 64, 48, None, (64, 100.0, None), 0.2), moe(4, 2, 16, 32))]},
}


def random_config(seed: int) -> dict:
    """A Pekodra configuration drawn from ``seed``: two to five layers, with either feed-forward or none, a loop
    anywhere or none, sizes that are and are not multiples of eight, windows from 1 to 500 positions."""
    import random

    r = random.Random(seed)
    width = r.choice([24, 40, 64, 66, 96, 136, 200, 256])
    layers = []
    for _ in range(r.randint(2, 5)):
        heads = r.choice([1, 2, 3, 4, 6, 8])
        kv_heads = r.choice([d for d in range(1, heads + 1) if heads % d == 0])
        dim = r.choice([6, 8, 12, 16, 24, 32, 40, 64, 96, 128])
        vdim = r.choice([4, 8, 10, 16, 24, 48, 64, 96, 160])
        rot = None
        if r.random() < 0.85:
            scaling = None
            if r.random() < 0.6:
                scaling = (r.choice([2.0, 4.0, 10.0]), r.choice([16, 64, 1024]), r.choice([32.0, 8.0, 2.0]),
                           r.choice([1.0, 0.5]))
            rot = (r.choice(range(2, dim + 1, 2)), r.choice([10.0, 1000.0, 500000.0]), scaling)
        window = r.choice([None, 1, 3, 16, 17, 50, 64, 120, 500])
        kind = r.random()
        if kind < 0.4:
            mlp = dense(r.choice([8, 40, 100, 256]))
        elif kind < 0.85:
            experts = r.choice([2, 3, 8, 12, 33])
            mlp = moe(experts, r.randint(1, min(experts, 4)), r.choice([8, 24, 32, 64, 96]),
                      r.choice([None, 16, 48, 96]))
        else:
            mlp = None
        layers.append(layer(attention(heads, kv_heads, dim, vdim, window, rot, r.choice([dim ** -0.5, 0.3, 0.07])), mlp))
    config = {"architecture": "Pekodra", "width": width, "vocab": r.randint(40, 700),
              "norm": {"eps": r.choice([1e-5, 1e-6])}, "embedding": {"scale": r.choice([1.0, 2.0, 0.5])},
              "logit_scale": r.choice([1.0, 0.5, 1.7]), "layers": layers}
    if r.random() < 0.8:
        start = r.randint(0, len(layers) - 1)
        config["loop"] = {"start": start, "stop": r.randint(start + 1, len(layers)), "times": r.randint(1, 3)}
    return config
