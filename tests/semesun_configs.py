"""Small Semesun configurations for the tests.  They differ from one another in every size; head counts, key and value sizes,
windows, table sizes and group counts are unequal on purpose, and some values that models tend to make equal or 1 are not
(and some are)."""
import copy


def attention(heads, kv_heads, dim, vdim, scale, window, keep_first, bias_max, bias_rows, v_mix=True):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max, "bias_rows": bias_rows,
         "mask": {"size": window, "keep_first": keep_first}}
    if v_mix is not None:
        m["v_mix"] = v_mix
    return m


def ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, ff, limit, count, keep, scale):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "identity": identity, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}


# Every kind of layer.  The blending layers keep values of 2 x 24 per token under unlike query head counts; one attention
# layer does not blend; windows of 70 and 33 with 3, 0 and 66 first tokens kept (66: more than a page); a layer without a
# feed-forward; three groups of which two stay; a router that takes one expert; a model whose first layer is recurrent.
SEM_A = {
    "architecture": "Semesun", "vocab": 160, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mamba2", "mixer": ssm(3, 20, 24, 1, 4, 1), "mlp": dense(112)},
        {"type": "attention", "mixer": attention(4, 2, 16, 24, 0.21, 70, 3, 200, 12), "mlp": moe(7, 2, 3, 40, 1.2, 3, 2, 1.5)},
        {"type": "attention", "mixer": attention(2, 1, 40, 8, 0.12, 33, 0, 90, 9, v_mix=False), "mlp": None},
        {"type": "attention", "mixer": attention(6, 2, 24, 24, 0.3, 70, 66, 64, 20), "mlp": moe(5, 0, 1, 24, 2.0, 1, 1, 1.0)},
        {"type": "mamba2", "mixer": ssm(4, 12, 10, 2, 2, 2), "mlp": moe(4, 2, 4, 16, 0.8, 2, 2, 2.5)},
    ],
}

# sizes the tensor-core kernels and the vector loads accept; attention first; several layers in one cache group
SEM_B = {
    "architecture": "Semesun", "vocab": 320, "width": 256, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": attention(8, 2, 32, 64, 0.17, 96, 5, 300, 12), "mlp": moe(8, 0, 2, 96, 1.25, 2, 1, 1.0)},
        {"type": "mamba2", "mixer": ssm(6, 32, 64, 2, 4, 2), "mlp": dense(384)},
        {"type": "attention", "mixer": attention(8, 2, 32, 64, 0.17, 96, 5, 300, 12), "mlp": moe(6, 2, 3, 64, 1.0, 4, 3, 2.0)},
        {"type": "attention", "mixer": attention(4, 2, 64, 64, 0.2, 40, 0, 50, 8), "mlp": dense(128)},
        {"type": "attention", "mixer": attention(8, 2, 32, 64, 0.17, 96, 5, 300, 12), "mlp": dense(64)},
    ],
}

# only recurrent layers: a model without any key/value cache
SEM_C = {
    "architecture": "Semesun", "vocab": 64, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mamba2", "mixer": ssm(1, 40, 33, 1, 3, 1), "mlp": None},
        {"type": "mamba2", "mixer": ssm(2, 8, 16, 2, 5, 4), "mlp": dense(64)},
    ],
}


def config(which):
    return copy.deepcopy({"a": SEM_A, "b": SEM_B, "c": SEM_C}[which])
