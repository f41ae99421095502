"""Plain, slow restatement of the Semesun decoder in numpy float64: whole sequences, no cache, no state carried between
calls, one function per mechanism, nothing imported from the package under test (the model-folder reader is the
tests' own).  The GPU tests compare the library with these functions.

Semesun lists its layers one by one.  A layer is a mixer, either windowed attention (query/key unit norm, a learned bias by
bucketed distance, a few first tokens that stay visible, values blended with those of the first such layer) or a Mamba-2
state-space mixer, followed by a feed-forward: a two-matrix unit with squared ReLU, or routed experts chosen group by group
with a correction that steers the choice but not the weights, and identity experts that pass their input through."""
from __future__ import annotations

import math

import numpy as np

from plain_llama import read_model  # noqa: F401  (config dict, name -> array)

D64 = np.float64


def rms_unit(x, eps):
    x = np.asarray(x, D64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, scale, eps):
    return rms_unit(x, eps) * np.asarray(scale, D64)


def lin(x, w):
    """Weights are stored [out, in]."""
    return np.asarray(x, D64) @ np.asarray(w, D64).T


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, D64)))


def silu(z):
    z = np.asarray(z, D64)
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, np.asarray(z, D64))


def relu_squared(z):
    return np.maximum(np.asarray(z, D64), 0.0) ** 2


# ----------------------------------------------------------------------------- attention

def distance_bucket(n, rows, far):
    """Row of the bias table for a distance n >= 0: one row per distance below rows // 2, then rows spaced evenly in the
    logarithm of the distance up to `far`, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def may_see(i, j, window, keep_first):
    """Whether the query at place i sees the key at place j."""
    return j <= i and (i - j < window or j < keep_first)


def attention_values(x, w, p, m):
    """This layer's own values [n, kv_heads, vdim], before any blending."""
    return lin(x, w[p + "v"]).reshape(x.shape[0], m["kv_heads"], m["vdim"])


def attention(x, w, p, m, eps, v_first=None, return_weights=False):
    """x [n, width] -> [n, width].  `v_first`: the values of the first blending layer, or None if this layer is it (or does
    not blend)."""
    n, H, G, dk, dv = x.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm(lin(x, w[p + "q"]).reshape(n, H, dk), w[p + "q.norm"], eps)
    k = rms_norm(lin(x, w[p + "k"]).reshape(n, G, dk), w[p + "k.norm"], eps)
    v = attention_values(x, w, p, m)
    if v_first is not None:
        lam = float(np.asarray(w[p + "vmix"], D64).reshape(()))
        v = (1.0 - lam) * v + lam * v_first
    rel = np.asarray(w[p + "rel"], D64) if p + "rel" in w else None      # (a part without a table: no bias)
    rows = rel.shape[0] if rel is not None else 0
    window, keep = m["mask"]["size"], m["mask"]["keep_first"]
    out = np.zeros((n, H, dv), D64)
    weights = np.zeros((H, n, n), D64)
    for h in range(H):
        g = h // (H // G)
        for i in range(n):
            js = [j for j in range(i + 1) if may_see(i, j, window, keep)]
            s = np.array([q[i, h] @ k[j, g] * m["scale"] + (rel[distance_bucket(i - j, rows, m["bias_max"]), h] if rows else 0.0) for j in js])
            e = np.exp(s - s.max())
            a = e / e.sum()
            weights[h, i, js] = a
            out[i, h] = a @ v[js, g]
    y = lin(out.reshape(n, H * dv), w[p + "o"])
    return (y, weights) if return_weights else y


# ----------------------------------------------------------------------------- Mamba-2

def causal_conv(u, taps, bias):
    """u [n, channels]; taps [channels, k] with the last column at the current token; zeros before the start."""
    u, taps = np.asarray(u, D64), np.asarray(taps, D64)
    n, k = u.shape[0], taps.shape[1]
    padded = np.concatenate([np.zeros((k - 1, u.shape[1]), D64), u])
    out = np.zeros_like(u)
    for j in range(k):
        out += padded[j:j + n] * taps[:, j]
    return out + np.asarray(bias, D64)


def mamba2(x, w, p, m, eps, return_state=False):
    """x [n, width] -> [n, width]: the state-space recurrence written out token by token."""
    n, H, P, N, G = x.shape[0], m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = lin(x, w[p + "in"])
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    xs = xbc[:, :inner].reshape(n, H, P)
    Bm = xbc[:, inner:inner + G * N].reshape(n, G, N)
    Cm = xbc[:, inner + G * N:].reshape(n, G, N)
    dt = softplus(dt + np.asarray(w[p + "dt_bias"], D64))
    decay_rate = -np.exp(np.asarray(w[p + "A_log"], D64))
    skip = np.asarray(w[p + "D"], D64)
    S = np.zeros((H, N, P), D64)
    y = np.zeros((n, H, P), D64)
    for t in range(n):
        for h in range(H):
            g = h // (H // G)
            S[h] = math.exp(decay_rate[h] * dt[t, h]) * S[h] + dt[t, h] * np.outer(Bm[t, g], xs[t, h])
            y[t, h] = S[h].T @ Cm[t, g] + skip[h] * xs[t, h]
    y = y.reshape(n, inner) * silu(z)
    parts = m["norm_groups"]
    y = rms_unit(y.reshape(n, parts, inner // parts), eps).reshape(n, inner) * np.asarray(w[p + "norm"], D64)
    out = lin(y, w[p + "o"])
    return (out, S) if return_state else out


# ----------------------------------------------------------------------------- feed-forward

def dense(x, w, p):
    return lin(relu_squared(lin(x, w[p + "up"])), w[p + "down"])


def route(x, w, p, r):
    """Per token: the chosen outputs of the router (index >= experts: an identity expert) and their weights."""
    E, I, top = r["experts"], r.get("identity", 0), r["top"]
    z = lin(x, w[p + "router"])
    e = np.exp(z - z.max(axis=-1, keepdims=True))
    s = e / e.sum(axis=-1, keepdims=True)
    choice = s + np.asarray(w[p + "correction"], D64)
    count, keep = r["groups"]["count"], r["groups"]["keep"]
    per = (E + I) // count
    chosen, weights = [], []
    for t in range(x.shape[0]):
        c = choice[t].copy()
        best = c.reshape(count, per).max(axis=1)
        kept = np.argsort(-best, kind="stable")[:keep]
        for g in range(count):
            if g not in kept:
                c[g * per:(g + 1) * per] = -np.inf
        idx = np.argsort(-c, kind="stable")[:top]
        chosen.append(idx)
        weights.append(s[t, idx] * r["scale"])
    return np.array(chosen), np.array(weights)


def expert(x, w, p, limit):
    g = np.minimum(lin(x, w[p + "gate"]), limit)
    u = np.clip(lin(x, w[p + "up"]), -limit, limit)
    return lin(g * sigmoid(1.702 * g) * (u + 1.0), w[p + "down"])


def routed_experts(x, w, p, mlp):
    r = mlp["router"]
    chosen, weights = route(x, w, p, r)
    out = np.zeros_like(np.asarray(x, D64))
    for t in range(x.shape[0]):
        for e, a in zip(chosen[t], weights[t]):
            if e >= r["experts"]:
                out[t] += a * np.asarray(x[t], D64)
            else:
                out[t] += a * expert(x[t:t + 1], w, f"{p}e{e}.", mlp["expert"]["limit"])[0]
    return out


def feed_forward(x, w, p, mlp):
    if mlp["kind"] == "dense":
        return dense(x, w, p)
    return routed_experts(x, w, p, mlp)


# ----------------------------------------------------------------------------- the model

def forward_logits(cfg, w, tokens, residuals=None):
    """Logits [n, vocab] of a whole sequence.  `residuals`: a list that receives the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = np.asarray(w["embed"], D64)[np.asarray(tokens)]
    v_first = None
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        m = layer["mixer"]
        if layer["type"] == "attention":
            if m.get("v_mix"):
                if v_first is None:
                    x = x + attention(h, w, p + "mix.", m, eps)
                    v_first = attention_values(h, w, p + "mix.", m)
                else:
                    x = x + attention(h, w, p + "mix.", m, eps, v_first=v_first)
            else:
                x = x + attention(h, w, p + "mix.", m, eps)
        elif layer["type"] == "mamba2":
            x = x + mamba2(h, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            x = x + feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
        if residuals is not None:
            residuals.append(x.copy())
    return lin(rms_norm(x, w["final.norm"], eps), w["head"])


def generate_greedy(cfg, w, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward_logits(cfg, w, tokens)[-1])))
    return tokens[len(prompt):]
