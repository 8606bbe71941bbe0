"""Host-side pieces of the Balenex design: the config reader (every size and constant from config.json, refusals) and
the oracle's own mechanisms against closed forms."""
import ctypes as C
import json
import math

import torch

from oracle import balenex as ob


def spec_of(kge, path):
    L = kge.lib()
    h = L.kge_model_open(str(path).encode())
    assert h, L.kge_last_error()
    buf = C.create_string_buffer(1 << 16)
    assert L.kge_model_spec_json(h, buf, 1 << 16) > 0
    L.kge_model_close(h)
    return json.loads(buf.value)


def test_config_reader_takes_every_size_and_constant(kge, tmp_path):
    layers = [ob.attention_layer(heads=6, kv_heads=3, dim=5, vdim=7, size=19, pool=4, scale=0.41, ff=13),
              ob.parallel_layer(heads=4, kv_heads=1, dim=10, vdim=6, conv=5, size=23, keep_first=2, rot_dims=6, base=777.0, scale=0.37, r_heads=3, r_dim=7, r_vdim=9, tau=12.5, ff=0)]
    cfg = ob.make_config(layers, vocab=77, width=40, groups=5, eps=3e-4)
    ob.save_model_dir(str(tmp_path), cfg, ob.make_weights(cfg))
    spec = spec_of(kge, tmp_path)
    assert (spec["model_type"], spec["vocab"], spec["d"], spec["L"]) == ("balenex", 77, 40, 2) and spec["has_weights"]
    assert abs(spec["eps"] - 3e-4) < 1e-9 and spec["norm_groups"] == 5 and spec["postnorm"]
    a, b = spec["layers"]
    assert (a["mixer"], a["heads"], a["kv_heads"], a["dim"], a["vdim"], a["window"], a["pool"], a["keep_first"]) == (6, 6, 3, 5, 7, 19, 4, 0)
    assert abs(a["scale"] - 0.41) < 1e-6 and (a["head_norm"], a["rot_dims"], a["v_rot"]) == (1, 0, 0)
    assert (a["mlp"], a["ff"], a["ff_silu_bias"]) == (1, 13, 1)
    assert (b["mixer"], b["heads"], b["kv_heads"], b["dim"], b["vdim"], b["conv"], b["window"], b["keep_first"], b["pool"]) == (5, 4, 1, 10, 6, 5, 23, 2, 0)
    assert (b["rot_dims"], b["rot_base"], b["rot_halves"], b["v_rot"], b["head_norm"]) == (6, 777.0, 1, 1, 1) and abs(b["scale"] - 0.37) < 1e-6
    assert (b["m_heads"], b["m_dim"], b["m_vdim"], b["mlp"]) == (3, 7, 9, 0) and abs(b["tau"] - 12.5) < 1e-6


def test_config_reader_refusals(kge, tmp_path):
    L = kge.lib()

    def refused(change, text):
        cfg = ob.make_config([ob.parallel_layer(), ob.attention_layer()])
        change(cfg)
        with open(tmp_path / "config.json", "w") as fh:
            json.dump(cfg, fh)
        assert not L.kge_model_open(str(tmp_path).encode())
        assert text in L.kge_last_error(), L.kge_last_error()
    refused(lambda c: c["layers"][0].update(type="wkv"), b"unknown layer type")
    refused(lambda c: c["norm"].update(groups=5), b"groups")
    refused(lambda c: c["layers"][0]["mixer"].pop("right"), b"'left' and 'right'")
    refused(lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=3), b"rotary")
    refused(lambda c: c["layers"][0]["mixer"]["left"].update(vdim=5), b"vdim")
    refused(lambda c: c["layers"][0]["mixer"]["left"]["mask"].update(size=0), b"attention side")
    refused(lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3), b"attention side")
    refused(lambda c: c["layers"][0]["mixer"]["right"].update(tau=0.0), b"linear-attention side")
    refused(lambda c: c["layers"][1]["mixer"]["mask"].update(pool=0), b"mask.pool")
    refused(lambda c: c["layers"][1]["mlp"].update(kind="moe"), b"moe")


def test_oracle_group_norm():
    x = torch.randn(3, 12, dtype=ob.DT)
    g = torch.randn(12, dtype=ob.DT)
    y = ob.group_norm(x, g, 3, 0.0)
    for p in range(3):      # every part has unit mean square before the weight
        assert torch.allclose((y[:, 4 * p:4 * p + 4] / g[4 * p:4 * p + 4]).pow(2).mean(-1), torch.ones(3, dtype=ob.DT))
    assert torch.allclose(ob.group_norm(x, g, 1, 1e-5), ob.rms(x, 1e-5, g))
    # a part that is scaled alone leaves the other parts as they are and (eps = 0) itself too
    x2 = x.clone()
    x2[:, 4:8] *= 7.0
    assert torch.allclose(ob.group_norm(x2, g, 3, 0.0), y)


def test_oracle_short_conv():
    u = torch.randn(6, 2, dtype=ob.DT)
    w = torch.tensor([[0.5, 2.0, -1.0], [0.0, 0.0, 1.0]], dtype=ob.DT)
    y = ob.short_conv(u, w)
    assert torch.allclose(y[:, 1], u[:, 1])      # only the last tap: the current token
    assert torch.allclose(y[0, 0], -u[0, 0]) and torch.allclose(y[1, 0], 2.0 * u[0, 0] - u[1, 0])
    assert torch.allclose(y[5, 0], 0.5 * u[3, 0] + 2.0 * u[4, 0] - u[5, 0])


def test_oracle_turn_halves_is_a_rotation_and_keeps_the_rest():
    x = torch.randn(5, 6, dtype=ob.DT)
    y = ob.turn_halves(x, list(range(5)), 100.0, 4)
    assert torch.equal(y[:, 4:], x[:, 4:]) and torch.allclose(y[0], x[0])
    assert torch.allclose(y[:, :4].pow(2).sum(-1), x[:, :4].pow(2).sum(-1))
    # position 3, pair (1, 3) turns by 3 * 100^(-2/4) = 0.3
    a, b = x[3, 1], x[3, 3]
    assert torch.allclose(y[3, 1], a * math.cos(0.3) - b * math.sin(0.3)) and torch.allclose(y[3, 3], b * math.cos(0.3) + a * math.sin(0.3))
    assert torch.allclose(ob.turn_halves(y, list(range(5)), 100.0, 4, sign=-1.0), x)
    # scores of turned vectors depend on the distance only
    q, k = torch.randn(1, 4, dtype=ob.DT), torch.randn(1, 4, dtype=ob.DT)
    s = [float(ob.turn_halves(q, [p + 7], 30.0, 4) @ ob.turn_halves(k, [p], 30.0, 4).T) for p in (0, 5, 40)]
    assert abs(s[0] - s[1]) < 1e-12 and abs(s[0] - s[2]) < 1e-12


def test_oracle_window_and_kept_tokens():
    assert [j for j in range(12) if ob.window_keep_visible(9, j, 3, 2)] == [0, 1, 7, 8, 9]
    assert [j for j in range(12) if ob.window_keep_visible(2, j, 3, 2)] == [0, 1, 2]
    assert [j for j in range(12) if ob.window_keep_visible(9, j, 3, 0)] == [7, 8, 9]
    m = ob.parallel_layer(heads=2, kv_heads=1, dim=4, vdim=4, size=3, keep_first=2, rot_dims=0)["mixer"]["left"]
    q, k = torch.randn(10, 2, 4, dtype=ob.DT), torch.randn(10, 1, 4, dtype=ob.DT)
    w = ob.left_weights(q, k, m, 1)
    assert torch.allclose(w.sum(-1), torch.ones(10, dtype=ob.DT))
    assert float(w[9, 2:7].abs().max()) == 0.0 and float(w[9, [0, 1, 7, 8, 9]].min()) > 0.0


def test_oracle_rotated_values_come_back_relative():
    """With one visible key the head's output is that key's value turned by the distance between key and query: the
    value is stored turned by its own position and the output is turned back by the query's."""
    v = torch.randn(1, 6, dtype=ob.DT)
    stored = ob.turn_halves(v, [4], 50.0, 6)
    out = ob.turn_halves(stored, [11], 50.0, 6, sign=-1.0)
    assert torch.allclose(out, ob.turn_halves(v, [-7], 50.0, 6))
    assert torch.allclose(ob.turn_halves(ob.turn_halves(v, [9], 50.0, 6), [9], 50.0, 6, sign=-1.0), v)


def test_oracle_gla_closed_form():
    """Two tokens, one head: o_0 = (q_0 . k_0) v_0, o_1 = (q_1 . (alpha_1 * k_0)) v_0 + (q_1 . k_1) v_1; the state after two
    tokens is diag(alpha_1) k_0 v_0^T + k_1 v_1^T; the decay lies in (0, 1) and tau = 1 gives the plain sigmoid."""
    m = {"heads": 1, "dim": 4, "vdim": 3, "tau": 4.0}
    cfg = ob.make_config([{"type": "parallel", "mixer": {"left": ob.parallel_layer()["mixer"]["left"], "right": m}, "mlp": None}], width=6, groups=1)
    P = ob.sub(ob.make_weights(cfg, seed=2), "l0.mix.right.")
    P["norm"] = torch.ones(3, dtype=ob.DT)
    P["o"] = torch.eye(6, 3, dtype=ob.DT)
    h = torch.randn(2, 6, dtype=ob.DT)
    q, k, v = h @ P["q"].T / 2.0, h @ P["k"].T, h @ P["v"].T
    al = ob.gla_decay(h, P, m)
    assert float(al.min()) > 0.0 and float(al.max()) < 1.0
    assert torch.allclose(al, torch.sigmoid((h @ P["a1"].T) @ P["a2"].T + P["a2.b"]) ** 0.25)
    assert torch.allclose(ob.gla_decay(h, P, dict(m, tau=1.0)), torch.sigmoid((h @ P["a1"].T) @ P["a2"].T + P["a2.b"]))
    o0 = (q[0] @ k[0]) * v[0]
    o1 = (q[1] @ (al[1] * k[0])) * v[0] + (q[1] @ k[1]) * v[1]
    gate = torch.nn.functional.silu(h @ P["g"].T)
    want = torch.stack([ob.rms(o0, 1e-5), ob.rms(o1, 1e-5)]) * gate
    out, S = ob.gla(h, P, m, 1e-5, return_state=True)
    assert torch.allclose(out[:, :3], want) and float(out[:, 3:].abs().max()) == 0.0
    assert torch.allclose(S[0], al[1][:, None] * torch.outer(k[0], v[0]) + torch.outer(k[1], v[1]))


def test_oracle_pooled_blocks():
    # a block is seen once ALL of it has left the window: block b iff b * P + P - 1 <= t - size
    assert [ob.pooled_visible_blocks(t, 5, 3) for t in range(12)] == [0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 2, 2]
    assert [ob.pooled_visible_blocks(t, 1, 1) for t in range(4)] == [0, 1, 2, 3]
    m = ob.attention_layer(heads=2, kv_heads=1, dim=4, vdim=4, size=5, pool=3)["mixer"]
    q, k = torch.randn(12, 2, 4, dtype=ob.DT), torch.randn(12, 1, 4, dtype=ob.DT)
    wb, wt = ob.pooled_weights(q, k, m, 1, 9)
    assert wb.shape == (1,) and wt.shape == (5,) and abs(float(wb.sum() + wt.sum()) - 1.0) < 1e-12      # positions 3 and 4 are not seen at all
    # equal keys everywhere: blocks and tokens weigh the same
    wb, wt = ob.pooled_weights(q, torch.ones(12, 1, 4, dtype=ob.DT), m, 0, 11)
    assert torch.allclose(torch.cat([wb, wt]), torch.full((7,), 1.0 / 7.0, dtype=ob.DT))


def test_oracle_one_token_and_layer_sums():
    """One token sees only itself: the pooled attention's output is the value projection through the output matrix, and a
    layer adds the normed sublayer results to the stream."""
    cfg = ob.make_config([ob.attention_layer(heads=2, kv_heads=2, dim=3, vdim=4)], width=8, groups=2)
    W = ob.make_weights(cfg, seed=4)
    P = ob.sub(W, "l0.mix.")
    eps, G = cfg["norm"]["eps"], 2
    x = W["embed"][torch.tensor([5])]
    h = ob.group_norm(x, W["l0.norm1"], G, eps)
    y = (h @ P["v"].T + P["v.b"]) @ P["o"].T + P["o.b"]
    assert torch.allclose(ob.pooled_attention(h, P, cfg["layers"][0]["mixer"], eps), y)
    x = x + ob.group_norm(y, W["l0.norm1b"], G, eps)
    h = ob.group_norm(x, W["l0.norm2"], G, eps)
    F = ob.sub(W, "l0.mlp.")
    f = (torch.nn.functional.silu(h @ F["gate"].T + F["gate.b"]) * (h @ F["up"].T + F["up.b"])) @ F["down"].T + F["down.b"]
    x = x + ob.group_norm(f, W["l0.norm2b"], G, eps)
    assert torch.allclose(ob.forward(cfg, W, [5]), ob.group_norm(x, W["final.norm"], G, eps) @ W["head"].T)
