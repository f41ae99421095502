"""Small Kogilix configurations for the tests.  They differ from one another in every size; head counts, head sizes, value
sizes and ranks are unequal on purpose, and some values that models tend to make equal or 1 are not (and some are)."""
import copy


def latent(heads, dim, vdim, q_rank, kv_rank, scale, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def matrix_lstm(heads, dim, vdim, gate_cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": gate_cap}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared_ff=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    m["shared"] = {"ff": shared_ff} if shared_ff else None
    return m


# every kind of layer, value sizes unlike key sizes, a layer without a feed-forward, one expert of several, all experts,
# a layer that reads another's latents with another head count; a latent of 40 values takes the generic attention kernel
KOG_A = {
    "architecture": "Kogilix", "vocab": 150, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mlstm", "mixer": matrix_lstm(2, 24, 40, 8.0), "mlp": dense(112)},
        {"type": "latent_attention", "mixer": latent(3, 32, 16, 48, 64, 0.2), "mlp": moe(5, 2, 40, 56)},
        {"type": "latent_attention", "mixer": latent(2, 16, 48, 24, 64, 0.3, kv_from=1), "mlp": None},
        {"type": "mlstm", "mixer": matrix_lstm(3, 16, 16, 15.0), "mlp": moe(4, 1, 24)},
        {"type": "latent_attention", "mixer": latent(1, 40, 40, 96, 40, 0.15), "mlp": moe(3, 3, 32, 16)},
    ],
}

# sizes the tensor-core attention kernels and the vector loads accept; attention first, two layers on one cache
KOG_B = {
    "architecture": "Kogilix", "vocab": 320, "width": 192, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "latent_attention", "mixer": latent(4, 32, 32, 96, 128, 0.18), "mlp": moe(8, 2, 96, 64)},
        {"type": "mlstm", "mixer": matrix_lstm(2, 64, 64, 10.0), "mlp": dense(256)},
        {"type": "latent_attention", "mixer": latent(6, 32, 64, 64, 128, 0.18, kv_from=0), "mlp": moe(8, 2, 96, 64)},
        {"type": "latent_attention", "mixer": latent(4, 32, 32, 96, 128, 0.18, kv_from=0), "mlp": dense(128)},
        {"type": "mlstm", "mixer": matrix_lstm(4, 32, 48, 12.0), "mlp": moe(6, 3, 64)},
    ],
}

# only recurrent layers: a model without any key/value cache
KOG_C = {
    "architecture": "Kogilix", "vocab": 64, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "mlstm", "mixer": matrix_lstm(1, 32, 8, 6.0), "mlp": None},
        {"type": "mlstm", "mixer": matrix_lstm(2, 8, 24, 20.0), "mlp": dense(64)},
    ],
}


def config(which):
    return copy.deepcopy({"a": KOG_A, "b": KOG_B, "c": KOG_C}[which])
