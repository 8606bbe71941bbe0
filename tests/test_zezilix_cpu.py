"""Host-side pieces of the Zezilix design: the config reader (every size and constant from config.json, the looped run
of layers unrolled onto shared tensors, refusals) and the oracle's own mechanisms against closed forms."""
import ctypes as C
import json
import math

import torch

from oracle import zezilix as oz


def spec_of(kge, path):
    L = kge.lib()
    h = L.kge_model_open(str(path).encode())
    assert h, L.kge_last_error()
    buf = C.create_string_buffer(1 << 16)
    assert L.kge_model_spec_json(h, buf, 1 << 16) > 0
    L.kge_model_close(h)
    return json.loads(buf.value)


def test_config_reader_takes_every_size_and_constant(kge, tmp_path):
    layers = [oz.wkv_layer(heads=3, dim=5, mlp="dense", ff=13, limit=2.25),
              oz.latent_layer(heads=4, dim=6, rot_dim=10, vdim=7, kv_rank=11, q_rank=9, base=777.0, scale=0.41, mlp="moe", experts=7, top=3, expert_ff=9, router_scale=1.25),
              oz.latent_layer(gated=True, heads=2, dim=8, rot_dim=4, vdim=12, kv_rank=5, mlp=None)]
    cfg = oz.make_config(layers, vocab=77, width=40, streams=3, residual_mult=0.35, loop=(1, 3, 2), eps=3e-4)
    oz.save_model_dir(str(tmp_path), cfg, oz.make_weights(cfg))
    spec = spec_of(kge, tmp_path)
    assert (spec["model_type"], spec["vocab"], spec["d"], spec["L"]) == ("zezilix", 77, 40, 5) and spec["has_weights"]
    assert abs(spec["eps"] - 3e-4) < 1e-9 and spec["streams"] == 3 and abs(spec["residual_mult"] - 0.35) < 1e-6 and spec["embed_norm"]
    a, b, c, b2, c2 = spec["layers"]
    assert (a["mixer"], a["heads"], a["dim"], a["mlp"], a["ff"]) == (3, 3, 5, 1, 13) and abs(a["ff_limit"] - 2.25) < 1e-6
    # a key counts its unrotated and rotated parts; the rotated part and the numbers of it that turn are listed apart
    assert (b["mixer"], b["heads"], b["kv_heads"], b["dim"], b["rot_part"], b["rot_dims"], b["vdim"], b["kv_rank"], b["q_rank"], b["out_gate"]) == (4, 4, 4, 16, 10, 10, 7, 11, 9, 0)
    assert abs(b["scale"] - 0.41) < 1e-6 and b["rot_base"] == 777.0
    assert (b["mlp"], b["experts"], b["top"], b["expert_ff"], b["route"], b["glu"]) == (2, 7, 3, 9, 2, 2) and abs(b["router_scale"] - 1.25) < 1e-6
    assert (c["mixer"], c["out_gate"], c["q_rank"], c["mlp"]) == (4, 1, 0, 0)
    # the run order 0, 1, 2, 1, 2: later passes run with the first pass's tensors
    assert [x["tensor_index"] for x in spec["layers"]] == [0, 1, 2, 1, 2]
    assert [x["weights_of"] for x in spec["layers"]] == [-1, -1, -1, 1, 2]
    assert (b2["heads"], b2["kv_rank"], c2["vdim"]) == (4, 11, 12)


def test_config_reader_loops(kge, tmp_path):
    layers = [oz.wkv_layer(mlp=None), oz.latent_layer(mlp=None), oz.wkv_layer(mlp=None)]
    for loop, order in [(None, [0, 1, 2]), ((0, 3, 2), [0, 1, 2, 0, 1, 2]), ((2, 3, 3), [0, 1, 2, 2, 2]), ((1, 1, 4), [0, 1, 2]), ((0, 1, 1), [0, 1, 2])]:
        cfg = oz.make_config(layers, loop=loop)
        assert oz.run_order(cfg) == order
        with open(tmp_path / "config.json", "w") as fh:
            json.dump(cfg, fh)
        assert [x["tensor_index"] for x in spec_of(kge, tmp_path)["layers"]] == order


def test_config_reader_refusals(kge, tmp_path):
    L = kge.lib()

    def refused(change, text):
        cfg = oz.make_config([oz.wkv_layer(mlp="dense"), oz.latent_layer(mlp="moe"), oz.latent_layer(gated=True, mlp=None)], loop=(0, 2, 2))
        change(cfg)
        with open(tmp_path / "config.json", "w") as fh:
            json.dump(cfg, fh)
        assert not L.kge_model_open(str(tmp_path).encode())
        assert text in L.kge_last_error(), L.kge_last_error()
    refused(lambda c: c["layers"][0].update(type="rglru"), b"unknown layer type")
    refused(lambda c: c["loop"].update(stop=4), b"loop")
    refused(lambda c: c["loop"].update(times=0), b"loop")
    refused(lambda c: c.update(streams=0), b"streams")
    refused(lambda c: c["layers"][1]["mixer"].pop("q_rank"), b"q_rank")
    refused(lambda c: c["layers"][1]["mixer"]["rot"].update(dims=3), b"latent-attention sizes")
    refused(lambda c: c["layers"][1]["mixer"].update(kv_rank=0), b"latent-attention sizes")
    refused(lambda c: c["layers"][0]["mlp"].pop("limit"), b"limit")
    refused(lambda c: c["layers"][1]["mlp"]["router"].update(top=9), b"moe sizes")


def test_oracle_turn_is_a_rotation_and_keeps_the_rest():
    x = torch.randn(5, 2, 6, dtype=oz.DT)
    y = oz.turn(x, torch.arange(5), 100.0, 4)
    assert torch.equal(y[..., 4:], x[..., 4:]) and torch.equal(y[0], x[0])
    assert torch.allclose(y[..., :4].pow(2).sum(-1), x[..., :4].pow(2).sum(-1))
    # position 3, pair 1 turns by 3 * 100^(-2/4) = 0.3
    a, b = x[3, 0, 2], x[3, 0, 3]
    assert torch.allclose(y[3, 0, 2], a * math.cos(0.3) - b * math.sin(0.3)) and torch.allclose(y[3, 0, 3], b * math.cos(0.3) + a * math.sin(0.3))
    # scores of turned vectors depend on the distance only
    q, k = torch.randn(1, 4, dtype=oz.DT), torch.randn(1, 4, dtype=oz.DT)
    s = [float(oz.turn(q, torch.tensor([p + 7]), 30.0, 4) @ oz.turn(k, torch.tensor([p]), 30.0, 4).T) for p in (0, 5, 40)]
    assert abs(s[0] - s[1]) < 1e-12 and abs(s[0] - s[2]) < 1e-12


def test_oracle_wkv_closed_form():
    """Two tokens, one head: o_0 = (r_0 . (u * k_0)) v_0 and o_1 = (r_1 . (w_1-free state k_0)) v_0 + (r_1 . (u * k_1)) v_1;
    the state after two tokens is diag(w_1) k_0 v_0^T + k_1 v_1^T."""
    m = {"heads": 1, "dim": 4}
    cfg = oz.make_config([{"type": "wkv", "mixer": m, "mlp": None}], width=6)
    P = oz.sub(oz.make_weights(cfg, seed=2), "l0.mix.")
    P["norm"] = torch.ones(4, dtype=oz.DT)
    P["o"] = torch.eye(6, 4, dtype=oz.DT)
    h = torch.randn(2, 6, dtype=oz.DT)
    prev = torch.stack([torch.zeros(6, dtype=oz.DT), h[0]])
    bl = {z: h + (prev - h) * P["mu." + z] for z in "rkvgw"}
    r, k, v = (bl[z] @ P[z].T for z in "rkv")
    w = torch.exp(-torch.exp(torch.tanh(bl["w"] @ P["w1"].T) @ P["w2"].T + P["w0"]))
    u = P["u"][0]
    o0 = (r[0] @ (u * k[0])) * v[0]
    o1 = (r[1] @ k[0]) * v[0] + (r[1] @ (u * k[1])) * v[1]
    gate = torch.nn.functional.silu(bl["g"] @ P["g"].T)
    want = torch.stack([oz.rms(o0, 1e-5), oz.rms(o1, 1e-5)]) * gate
    out, A = oz.wkv(h, P, m, 1e-5, return_state=True)
    assert torch.allclose(out[:, :4], want) and float(out[:, 4:].abs().max()) == 0.0
    assert torch.allclose(A[0], w[1][:, None] * torch.outer(k[0], v[0]) + torch.outer(k[1], v[1]))
    assert float(w.min()) > 0.0 and float(w.max()) < 1.0


def test_oracle_latent_attention_one_token_and_gate():
    """One token sees only itself: every head's output is its own value; the gate multiplies it before the output matrix."""
    L = oz.latent_layer(heads=2, dim=3, rot_dim=2, vdim=4, kv_rank=5, gated=True, mlp=None)
    cfg = oz.make_config([L], width=8)
    P = oz.sub(oz.make_weights(cfg, seed=4), "l0.mix.")
    h = torch.randn(1, 8, dtype=oz.DT)
    c = oz.rms((h @ P["dkv"].T)[:, :5], 1e-5, P["dkv.norm"])
    want = ((c @ P["uv"].T) * torch.sigmoid(h @ P["g"].T)) @ P["o"].T
    assert torch.allclose(oz.latent_attention(h, P, L["mixer"], 1e-5, True), want)
    p = oz.attention_weights(torch.randn(6, 8, dtype=oz.DT), P, L["mixer"], 1e-5, 1, 5)
    assert p.shape == (6,) and abs(float(p.sum()) - 1.0) < 1e-12


def test_oracle_streams_reduce_to_a_plain_residual():
    """One stream with unit read / write / mix weights and unit column scales: x <- x + m f(norm(x))."""
    cfg = oz.make_config([oz.wkv_layer(mlp="dense")], streams=1, residual_mult=0.6)
    W = oz.make_weights(cfg, seed=5)
    for k in W:
        if ".hc" in k or k.split(".")[-1] in ("ls1", "ls2"):
            W[k] = torch.ones_like(W[k])
    toks = [3, 9, 4, 4, 17]
    eps = cfg["norm"]["eps"]
    x = oz.rms(W["embed"][torch.tensor(toks)], eps, W["embed.norm"])
    x = x + 0.6 * oz.wkv(oz.rms(x, eps, W["l0.norm1"]), oz.sub(W, "l0.mix."), cfg["layers"][0]["mixer"], eps)
    x = x + 0.6 * oz.dense(oz.rms(x, eps, W["l0.norm2"]), oz.sub(W, "l0.mlp."), cfg["layers"][0]["mlp"]["limit"])
    assert torch.allclose(oz.forward(cfg, W, toks), oz.rms(x, eps, W["final.norm"]) @ W["head"].T)


def test_oracle_router_and_experts():
    f = {"expert": {"ff": 3}, "router": {"experts": 4, "top": 4, "scale": 2.0}}
    W = {"m.router": torch.randn(4, 6, dtype=oz.DT)}
    for e in range(4):
        W[f"m.e{e}.up"], W[f"m.e{e}.down"] = torch.randn(3, 6, dtype=oz.DT), torch.randn(6, 3, dtype=oz.DT)
    h = torch.randn(2, 6, dtype=oz.DT)
    s = oz.scores(h, W["m.router"])
    assert torch.allclose(s.sum(-1), torch.ones(2, dtype=oz.DT))
    want = sum(2.0 * s[:, e:e + 1] * (torch.relu(h @ W[f"m.e{e}.up"].T) ** 2 @ W[f"m.e{e}.down"].T) for e in range(4))
    assert torch.allclose(oz.moe(h, W, "m.", f), want)
    f["router"]["top"] = 1      # the weight stays the score of the full softmax: nothing is renormalised
    best = int(torch.argmax(s[0]))
    one = 2.0 * s[0, best] * (torch.relu(h[0] @ W[f"m.e{best}.up"].T) ** 2 @ W[f"m.e{best}.down"].T)
    assert torch.allclose(oz.moe(h, W, "m.", f)[0], one)
    assert math.isinf(float(oz.route_margins(h, W["m.router"], 4)[0])) and float(oz.route_margins(h, W["m.router"], 1)[0]) >= 0.0
