"""Oracle for the Zezilix design (a layer list of WKV recurrences and latent attention on a hyper-connected residual):
plain, slow float64 PyTorch, one function per mechanism.

TEST INFRASTRUCTURE.  Nothing here is shared with the product path.  Notation: t / j are positions from 0, W matrices
are [out, in] and act as h @ W.T, n(z, g) = z / sqrt(mean(z^2) + eps) * g.

  embedding    x = n(embed[token], g_embed); every one of the S residual copies X_1 .. X_S starts as x
  sublayer     (two per layer: 1 the mixer, 2 the feed-forward) with read weights a [S], write weights b [S], mix
               matrix M [S, S] (from, to), per-column scale c [D] and the model's multiplier m:
               y = f(n(sum_s a_s X_s, g));   X_j <- sum_s M[s, j] X_s + m b_j (c * y),   all j from the old copies
  loop         layers lo .. hi - 1 run `times` times in a row with the same tensors; every run has its own cache / state
  wkv          p = the previous position's h (zeros at t = 0);  blend_z = h + (p - h) mu_z for z in r, k, v, g, w;
               r, k, v = blend_z Wz (heads x dim), gate = silu(blend_g Wg),
               w = exp(-exp(tanh(blend_w W1) W2 + w0));  per head with state A [dim, dim] from zero:
               o_t = (A + diag(u) k_t v_t^T)^T r_t;  A <- diag(w_t) A + k_t v_t^T;
               out = ((o / sqrt(mean_head(o^2) + eps)) * g_norm * gate) Wo
  latent       c = n((h Wdkv)[:rank], g_kv), shared rotated key part kr = (h Wdkv)[rank:];  per head key = [c Wuk | rot(kr)],
               value = c Wuv;  query = [.. | rot(..)] of h Wq, or of n(h Wdq, g_q) Wuq;  rot turns pairs (2i, 2i + 1) of its
               first `dims` numbers by t base^(-2i / dims);  causal softmax of scale * q.k;  optional gate sigmoid(h Wg) on
               the heads' outputs; then Wo
  dense        a = min(h Wgate, L), b = clip(h Wup, -L, L);  (a sigmoid(1.702 a) (b + 1)) Wdown
  moe          s = softmax(h Wr) over all experts; the `top` largest s choose; out = sum_e scale s_e relu(h Wup_e)^2 Wdown_e
  logits       n(sum_s X_s, g_final) head^T
"""
from __future__ import annotations

import math

import torch

from .hybrid import DT, save_model_dir  # noqa: F401  (file writer only: config.json + safetensors by hand)


def wkv_layer(heads=2, dim=8, mlp="dense", **kw):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": _mlp(mlp, **kw)}


def latent_layer(heads=3, dim=8, rot_dim=4, vdim=6, kv_rank=10, q_rank=12, gated=False, base=3000.0, scale=0.3, rot_dims=None, mlp="moe", **kw):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if not gated:
        m["q_rank"] = q_rank
    return {"type": "latent_attention_2" if gated else "latent_attention", "mixer": m, "mlp": _mlp(mlp, **kw)}


def _mlp(kind, ff=20, limit=1.5, experts=5, top=2, expert_ff=12, router_scale=1.7):
    if kind is None:
        return None
    if kind == "dense":
        return {"kind": "dense", "ff": ff, "limit": limit}
    return {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top, "scale": router_scale}}


def make_config(layers, vocab=101, width=40, streams=2, residual_mult=0.4, loop=None, eps=1e-5):
    cfg = {"architecture": "Zezilix", "layers": layers, "norm": {"eps": eps}, "residual_mult": residual_mult, "streams": streams,
           "vocab": vocab, "width": width}
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


def run_order(cfg):
    n, lp = len(cfg["layers"]), cfg.get("loop")
    if not lp:
        return list(range(n))
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


def tensor_shapes(cfg, decay_rank=6):
    D, V, S = cfg["width"], cfg["vocab"], cfg["streams"]
    sh = {"embed": (V, D), "embed.norm": (D,), "final.norm": (D,), "head": (V, D)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for q in (1, 2) if L["mlp"] else (1,):
            sh.update({f"{p}norm{q}": (D,), f"{p}ls{q}": (D,), f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
        if L["type"] == "wkv":
            hd = m["heads"] * m["dim"]
            sh.update({p + "mix.mu." + z: (D,) for z in "rkvgw"})
            sh.update({p + "mix." + z: (hd, D) for z in "rkvg"})
            sh.update({p + "mix.w1": (decay_rank, D), p + "mix.w2": (hd, decay_rank), p + "mix.w0": (hd,), p + "mix.u": (m["heads"], m["dim"]),
                       p + "mix.norm": (hd,), p + "mix.o": (D, hd)})
        else:
            H, nq = m["heads"], m["heads"] * (m["dim"] + m["rot_dim"])
            if "q_rank" in m:
                sh.update({p + "mix.dq": (m["q_rank"], D), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (nq, m["q_rank"])})
            else:
                sh.update({p + "mix.q": (nq, D), p + "mix.g": (H * m["vdim"], D)})
            sh.update({p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], D), p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * m["dim"], m["kv_rank"]),
                       p + "mix.uv": (H * m["vdim"], m["kv_rank"]), p + "mix.o": (D, H * m["vdim"])})
        f = L["mlp"]
        if f and f["kind"] == "dense":
            sh.update({p + "mlp.gate": (f["ff"], D), p + "mlp.up": (f["ff"], D), p + "mlp.down": (D, f["ff"])})
        elif f:
            sh[p + "mlp.router"] = (f["router"]["experts"], D)
            for x in range(f["router"]["experts"]):
                sh.update({f"{p}mlp.e{x}.up": (f["expert"]["ff"], D), f"{p}mlp.e{x}.down": (D, f["expert"]["ff"])})
    return sh


def make_weights(cfg, seed=0, decay_rank=6):
    """Random bfloat16-representable weights (returned as float64) sized so that activations stay O(1), the decays spread
    over (0, 1), the clamps bite and the residual copies really differ."""
    g = torch.Generator().manual_seed(seed)
    S, W = cfg["streams"], {}
    for name, shape in tensor_shapes(cfg, decay_rank).items():
        last = name.split(".")[-1]
        r = lambda s=1.0: s * torch.randn(shape, generator=g)
        if last in ("norm", "norm1", "norm2"):
            t = 1.0 + 0.3 * r()
        elif last in ("ls1", "ls2"):
            t = 1.0 + 0.5 * r()
        elif last == "in":
            t = 1.0 / S + 0.3 * r()
        elif last == "out":
            t = 1.0 + 0.3 * r()
        elif last == "mix" and len(shape) == 2 and shape == (S, S) and ".hc" in name:
            t = torch.eye(S) * 0.8 + 0.2 / S + 0.1 * r()
        elif ".mu." in name:
            t = torch.rand(shape, generator=g)
        elif last == "w0":
            t = -1.0 + 1.5 * r()
        elif last == "u":
            t = 0.5 * r()
        elif name == "embed":
            t = r()
        elif last == "router":
            t = r(3.0 / math.sqrt(shape[-1]))
        elif last in ("w1", "w2"):
            t = r(2.0 / math.sqrt(shape[-1]))
        elif last in ("q", "uq", "uk", "dq", "dkv"):
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
    does: the distance between the oracle and the oracle with every stored activation - normed rows, blends, projection
    outputs, gated products, attention outputs, sublayer results - rounded to bfloat16 once.  A 16-bit engine computes
    another sample of this noise; tests hold it to a small multiple."""
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


def turn(x, positions, base, dims):
    """x [T, ..., n]: pairs (2i, 2i + 1) of the first `dims` numbers turn by position * base^(-2i / dims); the rest passes."""
    if dims == 0:
        return x
    out = x.clone()
    for t in range(x.shape[0]):
        for i in range(dims // 2):
            ang = float(positions[t]) * base ** (-2.0 * i / dims)
            a, b = x[t, ..., 2 * i], x[t, ..., 2 * i + 1]
            out[t, ..., 2 * i] = a * math.cos(ang) - b * math.sin(ang)
            out[t, ..., 2 * i + 1] = b * math.cos(ang) + a * math.sin(ang)
    return out


def latent_attention(h, P, m, eps, gated):
    T, H, dim, rd, vd, rank = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = _r(_r(rms(_r(h @ P["dq"].T), eps, P["dq.norm"])) @ P["uq"].T if "q_rank" in m else h @ P["q"].T).view(T, H, dim + rd)
    down = _r(h @ P["dkv"].T)
    c, kr = _r(rms(down[:, :rank], eps, P["dkv.norm"])), _r(turn(down[:, rank:], pos, m["rot"]["base"], m["rot"]["dims"]))
    kn, v = _r(c @ P["uk"].T).view(T, H, dim), _r(c @ P["uv"].T).view(T, H, vd)
    qn, qr = q[..., :dim], _r(turn(q[..., dim:], pos, m["rot"]["base"], m["rot"]["dims"]))
    out = torch.zeros(T, H, vd, dtype=DT)
    for hd in range(H):
        for t in range(T):
            s = (kn[:t + 1, hd] @ qn[t, hd] + kr[:t + 1] @ qr[t, hd]) * m["scale"]
            out[t, hd] = torch.softmax(s, 0) @ v[:t + 1, hd]
    out = _r(out.reshape(T, H * vd))
    if gated:
        out = _r(out * torch.sigmoid(_r(h @ P["g"].T)))
    return _r(out @ P["o"].T)


def attention_weights(h, P, m, eps, head, t):
    """The softmax weights of one head at position t (what a test reads to see which keys matter)."""
    T, H, dim, rd, rank = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (rms(h @ P["dq"].T, eps, P["dq.norm"]) @ P["uq"].T if "q_rank" in m else h @ P["q"].T).view(T, H, dim + rd)
    down = h @ P["dkv"].T
    c, kr = rms(down[:, :rank], eps, P["dkv.norm"]), turn(down[:, rank:], pos, m["rot"]["base"], m["rot"]["dims"])
    kn = (c @ P["uk"].T).view(T, H, dim)
    qr = turn(q[..., dim:], pos, m["rot"]["base"], m["rot"]["dims"])
    return torch.softmax((kn[:t + 1, head] @ q[t, head, :dim] + kr[:t + 1] @ qr[t, head]) * m["scale"], 0)


def wkv(h, P, m, eps, return_state=False):
    T, D = h.shape
    H, dim = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, D, dtype=DT), h[:-1]])
    blend = {z: _r(h + (prev - h) * P["mu." + z]) for z in "rkvgw"}
    r, k, v = (_r(blend[z] @ P[z].T).view(T, H, dim) for z in "rkv")
    gate = torch.nn.functional.silu(_r(blend["g"] @ P["g"].T))
    w = torch.exp(-torch.exp(_r(torch.tanh(blend["w"] @ P["w1"].T)) @ P["w2"].T + P["w0"])).view(T, H, dim)
    A = torch.zeros(H, dim, dim, dtype=DT)
    o = torch.zeros(T, H, dim, dtype=DT)
    for t in range(T):
        for hd in range(H):
            kv = torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = (A[hd] + P["u"][hd][:, None] * kv).T @ r[t, hd]
            A[hd] = w[t, hd][:, None] * A[hd] + kv
    out = _r(_r(rms(o, eps).reshape(T, H * dim) * P["norm"] * gate) @ P["o"].T)
    return (out, A) if return_state else out


def dense(h, P, limit):
    a = (h @ P["gate"].T).clamp(max=limit)
    b = (h @ P["up"].T).clamp(-limit, limit)
    return _r(_r(a * torch.sigmoid(1.702 * a) * (b + 1.0)) @ P["down"].T)


def scores(h, router):
    return torch.softmax(h @ router.T, -1)


def route_margins(h, router, top):
    """Per token: by how much the last chosen router logit leads the first one left out (inf when all are chosen)."""
    z, _ = torch.sort(h @ router.T, dim=-1, descending=True)
    if top >= z.shape[1]:
        return torch.full((h.shape[0],), math.inf, dtype=DT)
    return z[:, top - 1] - z[:, top]


def moe(h, W, prefix, f):
    s = scores(h, W[prefix + "router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in sorted(range(s.shape[1]), key=lambda e: (-s[t, e].item(), e))[:f["router"]["top"]]:
            a = _r(torch.relu(h[t] @ W[f"{prefix}e{e}.up"].T) ** 2)
            out[t] += f["router"]["scale"] * s[t, e] * _r(a @ W[f"{prefix}e{e}.down"].T)
    return out


def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def forward(cfg, W, tokens, return_layers=False, return_margins=False):
    """Logits [T, vocab] of one sequence (float64); optionally the sum of the residual copies after every layer run, or
    per token the smallest routing margin over the layer runs."""
    eps, m, S = cfg["norm"]["eps"], cfg["residual_mult"], cfg["streams"]
    x = rms(W["embed"][torch.tensor(tokens)], eps, W["embed.norm"])
    X = [x.clone() for _ in range(S)]
    layers, margins = [], torch.full((len(tokens),), math.inf, dtype=DT)
    for i in run_order(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        for q in (1, 2) if L["mlp"] else (1,):
            a, b, M = W[f"{p}hc{q}.in"], W[f"{p}hc{q}.out"], W[f"{p}hc{q}.mix"]
            h = _r(rms(sum(a[s] * X[s] for s in range(S)), eps, W[f"{p}norm{q}"]))
            if q == 1:
                P = sub(W, p + "mix.")
                y = wkv(h, P, L["mixer"], eps) if L["type"] == "wkv" else latent_attention(h, P, L["mixer"], eps, L["type"] == "latent_attention_2")
            elif L["mlp"]["kind"] == "dense":
                y = dense(h, sub(W, p + "mlp."), L["mlp"]["limit"])
            else:
                margins = torch.minimum(margins, route_margins(h, W[p + "mlp.router"], L["mlp"]["router"]["top"]))
                y = moe(h, W, p + "mlp.", L["mlp"])
            y = y * W[f"{p}ls{q}"]
            X = [sum(M[s, j] * X[s] for s in range(S)) + m * b[j] * y for j in range(S)]
        layers.append(sum(X))
    logits = _r(_r(rms(sum(X), eps, W["final.norm"])) @ W["head"].T)
    if return_margins:
        return logits, margins
    return (logits, layers) if return_layers else logits


def greedy(cfg, W, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(torch.argmax(forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]
