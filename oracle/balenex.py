"""Oracle for the Balenex design (a layer list of windowed attention beside gated linear attention, and of windowed
attention over pooled blocks, with grouped RMS norms before and after every sublayer): plain, slow float64 PyTorch, one
function per mechanism.

TEST INFRASTRUCTURE.  Nothing here is shared with the product path.  Notation: t / j are positions from 0, W matrices
are [out, in] and act as h @ W.T (+ b where a bias exists), n(z) = z / sqrt(mean(z^2) + eps).

  group norm   gn(x, g): x is cut into `groups` equal consecutive parts, each part divided by its own root mean square, times g
  layer        x <- x + gn(mixer(gn(x, g1)), g1b);  x <- x + gn(ff(gn(x, g2)), g2b)
  parallel     0.5 * (n(left(h)) * g_left + n(right(h)) * g_right)
    left       q, k, v = h Wz + bz;  each channel through a causal conv of `taps` weights (last tap on the current token);
               per head q <- n(q) g_q, k <- n(k) g_k;  the first rot.dims numbers of a head turn in pairs (i, i + dims / 2)
               by t * base^(-2i / dims);  values turn over ALL vdim numbers in pairs (m, m + vdim / 2) by their own position;
               j visible to t iff j <= t and (t - j < size or j < keep_first);  softmax(scale q.k);  the head's output turns back
               by -t;  then Wo
    right      q = h Wq / sqrt(dim), k = h Wk, v = h Wv, alpha = sigmoid((h Wa1^T) Wa2^T + ba2)^(1 / tau) per key channel;
               per head S <- diag(alpha_t) S + k_t v_t^T (S from zero), o_t = S^T q_t;  (n(o) g_norm per head) * silu(h Wg);  then Wo
  attention    q, k, v = h Wz + bz;  per head q <- n(q), k <- n(k) (no weight);  t sees j with 0 <= t - j < size, and one pooled
               key / value (the mean of the P keys / values of positions bP .. bP + P - 1) for every block b with
               bP + P - 1 <= t - size;  one softmax over tokens and blocks;  then Wo + bo
  dense        (silu(h Wgate + bgate) * (h Wup + bup)) Wdown + bdown
  logits       gn(x, g_final) head^T
"""
from __future__ import annotations

import math

import torch

from .hybrid import DT, save_model_dir  # noqa: F401  (file writer only: config.json + safetensors by hand)


def parallel_layer(heads=4, kv_heads=2, dim=8, vdim=6, conv=3, size=7, keep_first=2, rot_dims=4, base=100.0, scale=0.4,
                   r_heads=2, r_dim=6, r_vdim=8, tau=4.0, ff=20):
    left = {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"keep_first": keep_first, "size": size},
            "rot": {"base": base, "dims": rot_dims}, "scale": scale, "vdim": vdim}
    right = {"dim": r_dim, "heads": r_heads, "tau": tau, "vdim": r_vdim}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def attention_layer(heads=4, kv_heads=2, dim=8, vdim=6, size=7, pool=3, scale=0.5, ff=20):
    return {"type": "attention", "mixer": {"dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"pool": pool, "size": size}, "scale": scale, "vdim": vdim},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def make_config(layers, vocab=97, width=24, groups=3, eps=1e-5):
    return {"architecture": "Balenex", "layers": layers, "norm": {"eps": eps, "groups": groups}, "vocab": vocab, "width": width}


def tensor_shapes(cfg, decay_rank=5):
    D, V = cfg["width"], cfg["vocab"]
    sh = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for z in ("norm1", "norm1b") + (("norm2", "norm2b") if L["mlp"] else ()):
            sh[p + z] = (D,)
        if L["type"] == "parallel":
            a, r = m["left"], m["right"]
            nq, nk, nv = a["heads"] * a["dim"], a["kv_heads"] * a["dim"], a["kv_heads"] * a["vdim"]
            for z, n in (("q", nq), ("k", nk), ("v", nv)):
                sh.update({f"{p}mix.left.{z}": (n, D), f"{p}mix.left.{z}.b": (n,), f"{p}mix.left.{z}.conv": (n, a["conv"])})
            sh.update({p + "mix.left.q.norm": (a["dim"],), p + "mix.left.k.norm": (a["dim"],), p + "mix.left.o": (D, a["heads"] * a["vdim"])})
            rk, rv = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            sh.update({p + "mix.right.q": (rk, D), p + "mix.right.k": (rk, D), p + "mix.right.v": (rv, D), p + "mix.right.g": (rv, D),
                       p + "mix.right.o": (D, rv), p + "mix.right.norm": (r["vdim"],), p + "mix.right.a1": (decay_rank, D),
                       p + "mix.right.a2": (rk, decay_rank), p + "mix.right.a2.b": (rk,), p + "mix.left.out": (D,), p + "mix.right.out": (D,)})
        else:
            nq, nk, nv = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
            for z, n in (("q", nq), ("k", nk), ("v", nv)):
                sh.update({f"{p}mix.{z}": (n, D), f"{p}mix.{z}.b": (n,)})
            sh.update({p + "mix.o": (D, m["heads"] * m["vdim"]), p + "mix.o.b": (D,)})
        if L["mlp"]:
            f = L["mlp"]["ff"]
            sh.update({p + "mlp.gate": (f, D), p + "mlp.gate.b": (f,), p + "mlp.up": (f, D), p + "mlp.up.b": (f,), p + "mlp.down": (D, f), p + "mlp.down.b": (D,)})
    return sh


def make_weights(cfg, seed=0, decay_rank=5):
    """Random bfloat16-representable weights (returned as float64) sized so that activations stay O(1), the decays spread
    over (0, 1) and every bias and norm weight matters."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(cfg, decay_rank).items():
        last = name.split(".")[-1]
        r = lambda s=1.0: s * torch.randn(shape, generator=g)
        if last in ("norm", "norm1", "norm2", "norm1b", "norm2b", "out"):
            t = 1.0 + 0.3 * r()
        elif last == "b" and ".a2." in name:
            t = 2.0 + 2.0 * r()
        elif last == "b":
            t = 0.3 * r()
        elif last == "conv":
            t = 0.6 * r() + (torch.arange(shape[1]) == shape[1] - 1).to(torch.float32)
        elif name == "embed":
            t = r()
        elif last in ("a1", "a2"):
            t = r(2.0 / math.sqrt(shape[-1]))
        else:
            t = r(1.5 / math.sqrt(shape[-1]))
        W[name] = t.to(torch.bfloat16).to(DT)
    return W


# ------------------------------------------------------------------------------------------ mechanisms

ROUND = None      # a function applied to every stored activation: None for the exact oracle; see bfloat16_noise()


def _r(t):
    return t if ROUND is None else ROUND(t)


def bfloat16_noise(cfg, W, tokens):
    """Per position, the size (root mean square over the vocabulary, relative to the logits' size) of what rounding alone
    does: the distance between the oracle and the oracle with every stored activation - normed rows, projection and
    convolution outputs, cached keys and values, gated products, sublayer results - rounded to bfloat16 once."""
    global ROUND
    exact = forward(cfg, W, tokens)
    ROUND = lambda t: t.to(torch.bfloat16).to(DT)
    try:
        noisy = forward(cfg, W, tokens)
    finally:
        ROUND = None
    return ((noisy - exact).pow(2).mean(-1).sqrt() / exact.pow(2).mean().sqrt()).numpy()


def rms(z, eps, g=None):
    y = z / torch.sqrt(z.pow(2).mean(-1, keepdim=True) + eps)
    return y if g is None else y * g


def group_norm(x, g, groups, eps):
    T, D = x.shape
    return rms(x.reshape(T, groups, D // groups), eps).reshape(T, D) * g


def short_conv(u, w):
    """u [T, C]; w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def turn_halves(x, positions, base, dims, sign=1.0):
    """x [T, n]: the first `dims` numbers turn, i paired with i + dims / 2, by sign * position * base^(-2i / dims)."""
    if dims == 0:
        return x
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=DT)
    a = sign * torch.as_tensor(positions, dtype=DT)[:, None] * f[None, :]
    c, s = torch.cos(a), torch.sin(a)
    u, v = x[:, :half], x[:, half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[:, dims:]], dim=-1)


def window_keep_visible(t, j, size, keep_first):
    return j <= t and (t - j < size or j < keep_first)


def left_weights(q, k, m, head):
    """softmax weights [T, T] of one query head of the windowed attention (q, k after norm and rotation)."""
    T = q.shape[0]
    g = head // (m["heads"] // m["kv_heads"])
    s = m["scale"] * q[:, head] @ k[:, g].T
    t, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    vis = (j <= t) & ((t - j < m["mask"]["size"]) | (j < m["mask"]["keep_first"]))      # window_keep_visible, for all pairs
    return torch.softmax(s.masked_fill(~vis, -math.inf), dim=-1)


def left_qkv(h, P, m, eps):
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = list(range(T))
    q = _r(short_conv(_r(h @ P["q"].T + P["q.b"]), P["q.conv"])).reshape(T, H, dim)
    k = _r(short_conv(_r(h @ P["k"].T + P["k.b"]), P["k.conv"])).reshape(T, G, dim)
    v = _r(short_conv(_r(h @ P["v"].T + P["v.b"]), P["v.conv"])).reshape(T, G, vdim)
    q = rms(q, eps, P["q.norm"])
    k = rms(k, eps, P["k.norm"])
    q = _r(torch.stack([turn_halves(q[:, i], pos, m["rot"]["base"], m["rot"]["dims"]) for i in range(H)], 1))
    k = _r(torch.stack([turn_halves(k[:, i], pos, m["rot"]["base"], m["rot"]["dims"]) for i in range(G)], 1))
    v = _r(torch.stack([turn_halves(v[:, i], pos, m["rot"]["base"], vdim) for i in range(G)], 1))
    return q, k, v


def left_attention(h, P, m, eps):
    T = h.shape[0]
    H, G, vdim = m["heads"], m["kv_heads"], m["vdim"]
    q, k, v = left_qkv(h, P, m, eps)
    out = []
    for i in range(H):
        o = left_weights(q, k, m, i) @ v[:, i // (H // G)]
        out.append(turn_halves(o, list(range(T)), m["rot"]["base"], vdim, sign=-1.0))
    return _r(_r(torch.cat(out, dim=-1)) @ P["o"].T)


def gla_decay(h, P, m):
    z = _r(h @ P["a1"].T) @ P["a2"].T + P["a2.b"]
    return torch.sigmoid(z) ** (1.0 / m["tau"])


def gla(h, P, m, eps, return_state=False):
    T = h.shape[0]
    H, dim, vdim = m["heads"], m["dim"], m["vdim"]
    q = (_r(h @ P["q"].T) / math.sqrt(dim)).reshape(T, H, dim)
    k = _r(h @ P["k"].T).reshape(T, H, dim)
    v = _r(h @ P["v"].T).reshape(T, H, vdim)
    al = gla_decay(h, P, m).reshape(T, H, dim)
    S = torch.zeros(H, dim, vdim, dtype=DT)
    o = torch.zeros(T, H, vdim, dtype=DT)
    for t in range(T):
        S = al[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    y = (rms(o, eps, P["norm"])).reshape(T, H * vdim) * torch.nn.functional.silu(_r(h @ P["g"].T))
    out = _r(_r(y) @ P["o"].T)
    return (out, S) if return_state else out


def parallel_mixer(h, P, m, eps):
    a = left_attention(h, sub(P, "left."), m["left"], eps)
    b = gla(h, sub(P, "right."), m["right"], eps)
    return 0.5 * (rms(a, eps, P["left.out"]) + rms(b, eps, P["right.out"]))


def pooled_visible_blocks(t, size, pool):
    """how many pooled blocks position t sees: block b iff b * pool + pool - 1 <= t - size"""
    return max(0, (t - size + 1) // pool)


def pooled_weights(q, k, m, head, t):
    """softmax weights of query head `head` at position t: (over the pooled blocks it sees, over the tokens of its window);
    q, k after the norm."""
    g = head // (m["heads"] // m["kv_heads"])
    size, P = m["mask"]["size"], m["mask"]["pool"]
    nb, lo = pooled_visible_blocks(t, size, P), max(0, t - size + 1)
    kb = [_r(k[b * P:(b + 1) * P, g].mean(0)) for b in range(nb)]
    keys = torch.stack(kb + [k[j, g] for j in range(lo, t + 1)])
    w = torch.softmax(m["scale"] * keys @ q[t, head], dim=0)
    return w[:nb], w[nb:]


def pooled_attention(h, P, m, eps):
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, pool = m["mask"]["size"], m["mask"]["pool"]
    q = _r(rms(_r(h @ P["q"].T + P["q.b"]).reshape(T, H, dim), eps))
    k = _r(rms(_r(h @ P["k"].T + P["k.b"]).reshape(T, G, dim), eps))
    v = _r(h @ P["v"].T + P["v.b"]).reshape(T, G, vdim)
    out = torch.zeros(T, H, vdim, dtype=DT)
    for t in range(T):
        nb, lo = pooled_visible_blocks(t, size, pool), max(0, t - size + 1)
        for i in range(H):
            g = i // (H // G)
            wb, wt = pooled_weights(q, k, m, i, t)
            vb = [_r(v[b * pool:(b + 1) * pool, g].mean(0)) for b in range(nb)]
            vals = torch.stack(vb + [v[j, g] for j in range(lo, t + 1)])
            out[t, i] = torch.cat([wb, wt]) @ vals
    return _r(_r(out.reshape(T, H * vdim)) @ P["o"].T + P["o.b"])


def dense(h, P):
    a = _r(h @ P["gate"].T + P["gate.b"])
    b = _r(h @ P["up"].T + P["up.b"])
    return _r(_r(torch.nn.functional.silu(a) * b) @ P["down"].T + P["down.b"])


def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (float64); optionally the residual stream after every layer."""
    eps, G = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = W["embed"][torch.tensor(tokens)].clone()
    layers = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = _r(group_norm(x, W[p + "norm1"], G, eps))
        P = sub(W, p + "mix.")
        y = parallel_mixer(h, P, L["mixer"], eps) if L["type"] == "parallel" else pooled_attention(h, P, L["mixer"], eps)
        x = x + group_norm(y, W[p + "norm1b"], G, eps)
        if L["mlp"]:
            h = _r(group_norm(x, W[p + "norm2"], G, eps))
            x = x + group_norm(dense(h, sub(W, p + "mlp.")), W[p + "norm2b"], G, eps)
        layers.append(x.clone())
    logits = _r(_r(group_norm(x, W["final.norm"], G, eps)) @ W["head"].T)
    return (logits, layers) if return_layers else logits


def greedy(cfg, W, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]
