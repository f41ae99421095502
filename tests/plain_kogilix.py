"""Plain, slow restatement of the Kogilix decoder in numpy float64: whole sequences, no cache, no state carried between
calls, one function per mechanism, nothing imported from the package under test (the model-folder reader is the
tests' own).  The GPU tests compare the library with these functions."""
from __future__ import annotations

import numpy as np

from plain_llama import read_model  # noqa: F401  (config dict, name -> array)

D64 = np.float64


def rms_unit(x, eps):
    """x over the square root of (its mean square plus eps), along the last axis."""
    x = np.asarray(x, D64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, scale, eps):
    return rms_unit(x, eps) * np.asarray(scale, D64)


def lin(x, w):
    """Weights are stored [out, in]."""
    return np.asarray(x, D64) @ np.asarray(w, D64).T


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, D64)))


def gelu_tanh(z):
    z = np.asarray(z, D64)
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z):
    return np.maximum(np.asarray(z, D64), 0.0) ** 2


def log_sigmoid(z):
    return -np.logaddexp(0.0, -np.asarray(z, D64))


# ----------------------------------------------------------------------------- mixers

def latent_of(x, w, p, eps):
    """The key/value latent of every token: what a latent-attention layer remembers."""
    return rms_norm(lin(x, w[p + "dkv"]), w[p + "dkv.norm"], eps)


def latent_attention(x, w, p, m, eps, latent=None, return_weights=False):
    """x [n, width] -> [n, width].  Keys and values are made from the latent head by head; a query at place i sees j <= i.
    `latent`: another layer's latents to use instead of this layer's own."""
    n, H, dk, dv = x.shape[0], m["heads"], m["dim"], m["vdim"]
    cq = rms_norm(lin(x, w[p + "dq"]), w[p + "dq.norm"], eps)
    q = lin(cq, w[p + "uq"]).reshape(n, H, dk)
    c = latent_of(x, w, p, eps) if latent is None else latent
    k = lin(c, w[p + "uk"]).reshape(n, H, dk)
    v = lin(c, w[p + "uv"]).reshape(n, H, dv)
    out = np.zeros((n, H, dv), D64)
    weights = np.zeros((H, n, n), D64)
    for h in range(H):
        s = (q[:, h] @ k[:, h].T) * m["scale"]
        s = np.where(np.tril(np.ones((n, n), bool)), s, -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        pr = e / e.sum(axis=1, keepdims=True)
        weights[h] = pr
        out[:, h] = pr @ v[:, h]
    y = lin(out.reshape(n, H * dv), w[p + "o"])
    return (y, weights) if return_weights else y


def mlstm(x, w, p, m, eps, return_state=False):
    """The matrix memory, token by token from an empty state; the running maximum of the log gates starts at 0."""
    n, H, dk, dv, cap = x.shape[0], m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = lin(x, w[p + "q"]).reshape(n, H, dk) / np.sqrt(dk)
    k = lin(x, w[p + "k"]).reshape(n, H, dk)
    v = lin(x, w[p + "v"]).reshape(n, H, dv)
    gi = cap * np.tanh((lin(x, w[p + "i"]) + np.asarray(w[p + "i.b"], D64)) / cap)
    gf = log_sigmoid(cap * np.tanh((lin(x, w[p + "f"]) + np.asarray(w[p + "f.b"], D64)) / cap))
    S = np.zeros((H, dk, dv), D64)
    nn = np.zeros((H, dk), D64)
    mx = np.zeros(H, D64)
    o = np.zeros((n, H, dv), D64)
    for t in range(n):
        for h in range(H):
            m_new = max(gf[t, h] + mx[h], gi[t, h])
            keep, take = np.exp(gf[t, h] + mx[h] - m_new), np.exp(gi[t, h] - m_new)
            S[h] = keep * S[h] + take * np.outer(k[t, h], v[t, h])
            nn[h] = keep * nn[h] + take * k[t, h]
            mx[h] = m_new
            o[t, h] = (S[h].T @ q[t, h]) / (max(abs(nn[h] @ q[t, h]), np.exp(-m_new)) + 1e-6)
    y = rms_unit(o, eps).reshape(n, H * dv) * np.asarray(w[p + "norm"], D64) * sigmoid(lin(x, w[p + "g"]))
    y = lin(y, w[p + "o"])
    return (y, (S, nn, mx)) if return_state else y


# ----------------------------------------------------------------------------- feed-forwards

def gated_dense(x, w, p):
    return lin(gelu_tanh(lin(x, w[p + "gate"])) * lin(x, w[p + "up"]), w[p + "down"])


def route(x, w, p, top):
    """(chosen experts [n, top], their weights [n, top]): the largest logits, the lowest index first among equals; softmax
    over the chosen logits alone."""
    z = lin(x, w[p + "router"]) + np.asarray(w[p + "router.b"], D64)
    chosen = np.argsort(-z, axis=1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, chosen, axis=1)
    e = np.exp(zc - zc.max(axis=1, keepdims=True))
    return chosen, e / e.sum(axis=1, keepdims=True)


def routed_experts(x, w, p, mlp):
    x = np.asarray(x, D64)
    top = mlp["router"]["top"]
    chosen, weight = route(x, w, p, top)
    y = np.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(top):
            e = int(chosen[t, j])
            y[t] += weight[t, j] * lin(relu_squared(lin(x[t], w[p + f"e{e}.up"])), w[p + f"e{e}.down"])
    if mlp.get("shared"):
        y += sigmoid(lin(x, w[p + "shared.sg"])) * lin(relu_squared(lin(x, w[p + "shared.up"])), w[p + "shared.down"])
    return y


def feed_forward(x, w, p, mlp):
    return gated_dense(x, w, p) if mlp["kind"] == "dense" else routed_experts(x, w, p, mlp)


# ----------------------------------------------------------------------------- the model

def forward_logits(cfg, w, tokens, residuals=None):
    """Logits [n, vocab] of a whole sequence; `residuals`, a list, receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = np.asarray(w["embed"], D64)[np.asarray(tokens, np.int64)]
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        xn = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            latents[i] = latent_of(xn, w, p + "mix.", eps) if src is None else latents[src]
            x = x + latent_attention(xn, w, p + "mix.", m, eps, latent=latents[i])
        elif layer["type"] == "mlstm":
            x = x + mlstm(xn, w, p + "mix.", m, eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            x = x + feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
        if residuals is not None:
            residuals.append(x.copy())
    return lin(rms_norm(x, w["final.norm"], eps), w["head"])


def generate_greedy(cfg, w, prompt, n_new):
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(np.argmax(forward_logits(cfg, w, seq)[-1])))
    return seq[len(prompt):]
