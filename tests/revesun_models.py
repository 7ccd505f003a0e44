"""Tiny Revesun configurations for the tests: every size differs between them and between their layers, and the
values that make two mechanisms coincide (keys as wide as values, one kv head, one norm group, one tap) appear in
one layer and not in the next."""


def attention(heads, kv_heads, dim, vdim, conv, block, rot_dims, rot_base, scale, ff):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                      "mask": {"size": block}, "rot": {"dims": rot_dims, "base": rot_base}, "scale": scale},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def mingru(width, ff):
    return {"type": "mingru", "mixer": {"width": width}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


TINY_REVESUN = {
    # a recurrent layer first and with a feed-forward, attention without one, three norm groups, an odd vocabulary
    "p": {"architecture": "Revesun", "width": 48, "vocab": 131, "norm": {"eps": 1e-6, "groups": 3},
          "layers": [mingru(40, 72),
                     attention(6, 2, 16, 24, 3, 13, 8, 100.0, 0.3, None),
                     attention(4, 4, 20, 8, 2, 32, 20, 10000.0, 0.25, 64),
                     mingru(33, None)]},
    # one norm group, one tap (no convolution state), blocks shorter than a page, heads of 32 and 8
    "q": {"architecture": "Revesun", "width": 64, "vocab": 256, "norm": {"eps": 1e-5, "groups": 1},
          "layers": [attention(2, 1, 32, 32, 1, 5, 2, 7.0, 0.2, 96),
                     attention(4, 2, 8, 40, 5, 50, 6, 500.0, 0.4, 80)]},
    # a single layer of each kind, wide blocks (never left in short prompts), four groups
    "r": {"architecture": "Revesun", "width": 32, "vocab": 77, "norm": {"eps": 1e-4, "groups": 4},
          "layers": [attention(1, 1, 24, 16, 4, 1000, 24, 30.0, 0.15, None),
                     mingru(64, 48)]},
    # recurrent layers only: a model without a single page
    "s": {"architecture": "Revesun", "width": 40, "vocab": 64, "norm": {"eps": 1e-5, "groups": 2},
          "layers": [mingru(24, None), mingru(56, 32)]},
}


def random_config(seed: int) -> dict:
    """A Revesun configuration drawn from ``seed``: two to five layers of either kind in any order, with or without
    a feed-forward, sizes that are and are not multiples of eight, one to six taps, blocks from 3 to 500 positions."""
    import random

    r = random.Random(seed)
    width = r.choice([24, 40, 64, 66, 96, 136, 200, 256, 320])
    groups = r.choice([g for g in range(1, 9) if width % g == 0])
    layers = []
    for _ in range(r.randint(2, 5)):
        ff = r.choice([None, r.choice([8, 40, 100, 256, 513])])
        if r.random() < 0.6:
            heads = r.choice([1, 2, 3, 4, 6, 8])
            kv_heads = r.choice([d for d in range(1, heads + 1) if heads % d == 0])
            dim = r.choice([6, 8, 12, 16, 24, 32, 40, 64, 96, 128])
            vdim = r.choice([4, 8, 10, 16, 24, 48, 64, 96, 160, 256])
            layers.append(attention(heads, kv_heads, dim, vdim, r.randint(1, 6), r.choice([3, 16, 17, 50, 64, 120, 500]),
                                    r.choice(range(0, dim + 1, 2)), r.choice([10.0, 1000.0, 50000.0]),
                                    r.choice([dim ** -0.5, 0.3, 0.07]), ff))
        else:
            layers.append(mingru(r.choice([8, 30, 64, 100, 257]), ff))
    return {"architecture": "Revesun", "width": width, "vocab": r.randint(40, 700),
            "norm": {"eps": r.choice([1e-5, 1e-6]), "groups": groups}, "layers": layers}
