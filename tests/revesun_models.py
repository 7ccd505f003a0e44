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
