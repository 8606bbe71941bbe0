"""The Zezilix design in the engine against the plain float64 oracle (oracle/zezilix.py): every mechanism alone, whole
prompts against pieces and token-by-token decoding, mixed batches, reused pages and state slots, far keys and page
borders with peaked scores, slowly decaying recurrent memory, the first tokens, long decoding, other sizes, looped
layers, and greedy generation through the scheduler.  float32 engines give the sharp comparison; bfloat16 ones are held
to a rounding-sized bound."""
import copy

import numpy as np
import pytest
import torch

from oracle import zezilix as oz

pytestmark = pytest.mark.gpu


def make_engine(kge, tmp_path, cfg, W, dtype="float32", tokens=512, bs=16, seqs=4, name="m", batched=0):
    d = str(tmp_path / name)
    oz.save_model_dir(d, cfg, W)
    nb = (tokens + bs - 1) // bs
    return kge.LLM(d, dtype=dtype, block_size=bs, num_gpu_blocks_override=nb + 1, max_model_len=nb * bs + 1, max_num_seqs=seqs,
                   max_num_batched_tokens=batched or nb * bs, enable_prefix_caching=False)


def run_pieces(llm, rid, tokens, pieces):
    """Feed `tokens` in steps of the given sizes, asking for every position's logits."""
    out, at = [], 0
    for n in pieces:
        llm.trace_add(rid, tokens[at:at + n])
        out.append(llm.trace_step([(rid, n, list(range(n)))]))
        at += n
    assert at == len(tokens)
    return np.concatenate(out)


def check(got, want, dtype, what="", margins=None, noise=None, f32=2e-4):
    """Row-wise error against the oracle, relative to the logits' size.  float32 engines are held to 2e-4.  bfloat16
    engines are held to 4e-2, or, where the case gives `noise` (oz.bfloat16_noise: what rounding alone does in the oracle,
    per row), to three times the noise that nine rows in ten stay below; rounding noise has a heavy tail (a squared
    activation next to zero, a router logit next to its neighbour), so one row in ten may pass that bound, up to three
    times the noisiest row of the oracle.  bfloat16 engines form the router's logits from rounded activations: where the
    oracle's own choice hangs on a margin below 0.05 (`margins`, per token) another expert may be chosen, so such rows are
    left out, and the rows after the first of them, which see that token through later layers' attention and recurrences,
    get a wider bound (a lost key, state or expert costs 0.3 and more).  The float32 runs of the same cases are the sharp ones."""
    want = want.numpy() if isinstance(want, torch.Tensor) else want
    scale = np.sqrt((want ** 2).mean())
    err = np.sqrt(((got - want) ** 2).mean(-1)) / scale
    b16 = max(4e-2, 3.0 * float(np.quantile(noise, 0.9))) if noise is not None else 4e-2
    lim = np.full(len(err), f32 if dtype == "float32" else b16)
    if dtype != "float32" and margins is not None:
        close = np.asarray(margins) < 0.05
        assert close.mean() < 0.5, f"{what}: {close.sum()} of {len(close)} rows hang on a close routing call"
        if close.any():
            lim[int(np.argmax(close)):] = max(0.25, b16)
            lim[close] = np.inf
    over = err >= lim
    if dtype != "float32" and noise is not None and over.any():
        worst = int(np.argmax(err / lim))
        assert over.mean() <= 0.1 and (err[over] < 3.0 * float(np.max(noise))).all(), \
            f"{what}: {over.sum()} of {len(err)} rows over {b16:.3g}, row {worst} is {err[worst]:.3g} of the logits' size"
        return
    worst = int(np.argmax(err / lim))
    assert not over.any(), f"{what}: row {worst} is {err[worst]:.3g} of the logits' size (limit {lim[worst]:.3g})"


def oracle(cfg, W, toks):
    lg, mg = oz.forward(cfg, W, toks, return_margins=True)
    return lg.numpy(), mg.numpy()


def prompt(cfg, n, seed=1):
    return torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def silence_mixers(W):
    for k in W:
        if k.endswith("mix.o"):
            W[k] = torch.zeros_like(W[k])
    return W


ALONE = {
    "wkv": dict(layers=[oz.wkv_layer(mlp=None)]),
    "wkv-one-head": dict(layers=[oz.wkv_layer(heads=1, dim=12, mlp=None)]),
    "wkv-plain-residual": dict(layers=[oz.wkv_layer(mlp=None)], streams=1, residual_mult=1.0),
    "latent": dict(layers=[oz.latent_layer(mlp=None)]),
    "latent-gated": dict(layers=[oz.latent_layer(gated=True, mlp=None)]),
    "latent-no-rotation": dict(layers=[oz.latent_layer(rot_dim=0, mlp=None)]),
    "latent-one-head": dict(layers=[oz.latent_layer(heads=1, vdim=9, mlp=None)]),
    "latent-three-streams": dict(layers=[oz.latent_layer(mlp=None)], streams=3),
    "dense": dict(layers=[oz.wkv_layer(mlp="dense", limit=0.6)]),
    "moe": dict(layers=[oz.wkv_layer(mlp="moe")]),
    "moe-top1": dict(layers=[oz.wkv_layer(mlp="moe", top=1, router_scale=1.0)]),
    "moe-all-experts": dict(layers=[oz.wkv_layer(mlp="moe", experts=3, top=3)]),
    "moe-top6-of-9": dict(layers=[oz.wkv_layer(mlp="moe", experts=9, top=6)]),
}


@pytest.mark.parametrize("mech", sorted(ALONE))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mechanism_alone(kge, tmp_path, mech, dtype):
    cfg = oz.make_config(**ALONE[mech])
    W = oz.make_weights(cfg, seed=3)
    if mech.startswith(("dense", "moe")):
        silence_mixers(W)
    toks = prompt(cfg, 45)
    want, mg = oracle(cfg, W, toks)
    if mech == "dense":      # the limit really cuts
        loose = copy.deepcopy(cfg)
        loose["layers"][0]["mlp"]["limit"] = 50.0
        assert float(np.abs(oz.forward(loose, W, toks).numpy() - want).max()) > 0.1
    llm = make_engine(kge, tmp_path, cfg, W, dtype)
    got = run_pieces(llm, 0, toks, [45])
    llm.close()
    check(got, want, dtype, mech, mg)


def full(**kw):
    """Every kind of layer, a looped run in the middle (layers 1 and 2 twice), a layer without feed-forward."""
    layers = [oz.wkv_layer(mlp="dense"), oz.latent_layer(gated=True, mlp="moe"), oz.latent_layer(heads=2, dim=6, rot_dim=6, vdim=8, kv_rank=7, q_rank=9, mlp="moe"),
              oz.wkv_layer(heads=3, dim=4, mlp="moe"), oz.latent_layer(gated=True, heads=2, mlp=None)]
    return oz.make_config(layers, loop=(1, 3, 2), **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_prefill_decode_and_pieces_agree_with_the_oracle(kge, tmp_path, dtype):
    cfg = full()
    W = oz.make_weights(cfg, seed=5)
    toks = prompt(cfg, 75)
    want, mg = oracle(cfg, W, toks)
    noise = oz.bfloat16_noise(cfg, W, toks)
    llm = make_engine(kge, tmp_path, cfg, W, dtype)
    for rid, pieces in enumerate([[75], [30] + [1] * 45, [1] * 75, [2, 3, 17, 2, 31, 5, 2, 2, 9, 2], [23, 2, 24, 26], [47, 2, 1, 1, 24]]):
        got = run_pieces(llm, rid, toks, pieces)
        llm.trace_end(rid)
        check(got, want, dtype, f"pieces {pieces[:6]}", mg, noise)
    llm.close()


def test_layer_outputs_match(kge, tmp_path):
    """The sum of the residual copies after every layer run; the looped layers run twice with the same tensors and a
    cache and state of their own."""
    cfg = full()
    W = oz.make_weights(cfg, seed=6)
    toks = prompt(cfg, 33)
    _, layers = oz.forward(cfg, W, toks, return_layers=True)
    assert len(layers) == 7
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    buf = np.zeros((7, 33, cfg["width"]), dtype=np.float32)
    llm.set_layer_dump(buf)
    run_pieces(llm, 0, toks, [20, 13])
    last = buf.reshape(-1)[:7 * 13 * cfg["width"]].reshape(7, 13, cfg["width"]).copy()      # the dump is packed per step: [run, row of the step, width]
    llm.set_layer_dump(None)
    llm.close()
    for i, x in enumerate(layers):      # the dump holds the last step's rows: positions 20 .. 32
        assert np.abs(last[i] - x.numpy()[20:]).max() < 2e-4 * float(x.abs().max()), f"layer run {i}"


def test_looped_layers_keep_their_own_cache_and_state(kge, tmp_path):
    """A model that runs its two layers three times differs from one that runs them once, and decoding it token by
    token (every run reading its own cache and state) equals the whole prompt."""
    layers = [oz.wkv_layer(mlp=None), oz.latent_layer(mlp=None)]
    cfg = oz.make_config(layers, loop=(0, 2, 3))
    W = oz.make_weights(cfg, seed=21)
    toks = prompt(cfg, 40, 5)
    want = oz.forward(cfg, W, toks)
    assert float((want - oz.forward(oz.make_config(layers), W, toks)).abs().max()) > 0.1
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    check(run_pieces(llm, 0, toks, [10] + [1] * 30), want, "float32")
    llm.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_of_unequal_requests(kge, tmp_path, dtype):
    cfg = full()
    W = oz.make_weights(cfg, seed=7)
    P = {0: prompt(cfg, 61, 10), 1: prompt(cfg, 9, 11), 2: prompt(cfg, 40, 12), 3: prompt(cfg, 1, 13)}
    want = {r: oracle(cfg, W, t) for r, t in P.items()}
    # each step: (request, number of tokens); prompt pieces beside single tokens, requests pausing and resuming
    steps = [[(0, 19), (1, 1), (3, 1)], [(1, 1), (2, 2), (0, 2)], [(0, 20), (1, 1)], [(2, 18), (1, 1), (0, 1)], [(1, 5), (2, 1)],
             [(0, 1), (2, 1)], [(0, 18), (2, 18)]]
    llm = make_engine(kge, tmp_path, cfg, W, dtype)
    at = {r: 0 for r in P}
    got = {r: [] for r in P}
    for st in steps:
        entries = []
        for r, n in st:
            llm.trace_add(r, P[r][at[r]:at[r] + n])
            entries.append((r, n, list(range(n))))
        lg = llm.trace_step(entries)
        k = 0
        for r, n in st:
            got[r].append(lg[k:k + n])
            k += n
            at[r] += n
    llm.close()
    for r in P:
        assert at[r] == len(P[r])
        check(np.concatenate(got[r]), want[r][0], dtype, f"request {r}", want[r][1], oz.bfloat16_noise(cfg, W, P[r]))


def test_pages_and_slots_are_used_again(kge, tmp_path):
    """Two state slots and a pool of 96 tokens: five requests pass through, each in pages and a slot that an earlier
    request filled; each must come out as if it had run alone (a slot's old matrix or saved row must not leak)."""
    cfg = full()
    W = oz.make_weights(cfg, seed=8)
    llm = make_engine(kge, tmp_path, cfg, W, "float32", tokens=96, bs=16, seqs=2)
    P = {r: prompt(cfg, n, 20 + r) for r, n in enumerate([40, 33, 47, 18, 30])}
    want = {r: oz.forward(cfg, W, t).numpy() for r, t in P.items()}
    got = {}
    got[0] = run_pieces(llm, 0, P[0], [40])
    llm.trace_add(1, P[1][:20])
    a = llm.trace_step([(1, 20, list(range(20)))])
    llm.trace_end(0)
    llm.trace_add(2, P[2])
    llm.trace_add(1, P[1][20:])
    b = llm.trace_step([(2, 30, list(range(30))), (1, 13, list(range(13)))])
    got[1] = np.concatenate([a, b[30:]])
    c = llm.trace_step([(2, 17, list(range(17)))])
    got[2] = np.concatenate([b[:30], c])
    llm.trace_end(1)
    got[3] = run_pieces(llm, 3, P[3], [2, 16])
    llm.trace_end(2)
    llm.trace_end(3)
    got[4] = run_pieces(llm, 4, P[4], [29, 1])
    llm.close()
    for r in P:
        check(got[r], want[r], "float32", f"request {r}")


def peaked(gated, heads, dim, rot_dim, vdim):
    """Latent attention alone with a large score scale: single keys carry most of a row's weight, so a key that is lost,
    misplaced in its page or turned by the wrong position moves the logits far beyond rounding."""
    return oz.make_config([oz.latent_layer(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=14, q_rank=16, gated=gated, scale=0.5, base=200.0, mlp=None)])


@pytest.mark.parametrize("shape", [(False, 3, 8, 4, 6), (True, 2, 16, 16, 24)])      # the per-row kernel; the tensor-core kernel (bfloat16, key size a multiple of 16)
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_keys_and_page_borders_with_peaked_scores(kge, tmp_path, dtype, shape):
    cfg = peaked(*shape)
    W = oz.make_weights(cfg, seed=9)
    toks = prompt(cfg, 330, 30)
    want = oz.forward(cfg, W, toks)
    # the setup shows what it should: without the first page's keys late rows move visibly, and late rows do give single far keys real weight
    late = oz.forward(cfg, W, toks[16:])[-30:]
    assert float((late - want[-30:]).abs().max()) > 0.2
    x = oz.rms(W["embed"][torch.tensor(toks)], cfg["norm"]["eps"], W["embed.norm"])
    h = oz.rms(sum(W["l0.hc1.in"][s] * x for s in range(cfg["streams"])), cfg["norm"]["eps"], W["l0.norm1"])
    far = 0
    for t in range(300, 330):
        p = oz.attention_weights(h, oz.sub(W, "l0.mix."), cfg["layers"][0]["mixer"], cfg["norm"]["eps"], 0, t)
        far += int(p[:t - 100].max() > 0.2)
    assert far >= 5
    llm = make_engine(kge, tmp_path, cfg, W, dtype, bs=16)
    check(run_pieces(llm, 0, toks, [330]), want, dtype, "whole")
    llm.trace_end(0)
    check(run_pieces(llm, 1, toks[:100], [15, 1, 1, 1, 14, 2, 30, 1, 1, 34]), want[:100], dtype, "pieces and single tokens across page borders")
    llm.trace_end(1)
    got = np.concatenate([run_pieces(llm, 2, toks[:290], [290]), run_pieces(llm, 2, toks[290:], [1] * 40)])
    check(got, want, dtype, "decoding far from the first keys")
    llm.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_recurrent_memory_that_decays_slowly(kge, tmp_path, dtype):
    """WKV alone with decays close to 1 (and a few fast channels): the matrix state remembers the first tokens for
    hundreds of positions, so a state that is lost, reset or carried over at the cut of a prompt shows at the end."""
    cfg = oz.make_config([oz.wkv_layer(heads=2, dim=16, mlp=None)], width=32)
    W = oz.make_weights(cfg, seed=10)
    W["l0.mix.w0"] = torch.where(torch.arange(32) % 5 == 0, 0.5, -5.0).to(oz.DT)
    W["l0.mix.w2"] = W["l0.mix.w2"] * 0.25
    toks = prompt(cfg, 260, 31)
    want = oz.forward(cfg, W, toks)
    other = oz.forward(cfg, W, prompt(cfg, 8, 32) + toks[8:])
    assert float((other[-20:] - want[-20:]).abs().max()) > 0.05      # the first tokens still matter 250 positions later
    llm = make_engine(kge, tmp_path, cfg, W, dtype)
    check(run_pieces(llm, 0, toks, [260]), want, dtype, "whole")
    llm.trace_end(0)
    check(run_pieces(llm, 1, toks, [63, 2, 1, 64, 2, 97, 1, 30]), want, dtype, "pieces")
    llm.trace_end(1)
    check(run_pieces(llm, 2, toks, [200] + [1] * 60), want, dtype, "decoding")
    llm.close()


def test_tensor_core_sizes(kge, tmp_path):
    """bfloat16 at sizes the tensor-core paths take: 16-byte rows everywhere, key sizes that are multiples of 16,
    64-token pages, prompts long enough for the 64-row attention CTAs, feed-forward widths that are multiples of 64."""
    layers = [oz.wkv_layer(heads=2, dim=32, mlp="dense", ff=128), oz.latent_layer(heads=4, dim=32, rot_dim=16, vdim=40, kv_rank=32, gated=True, mlp="moe", expert_ff=64, experts=4),
              oz.latent_layer(heads=2, dim=16, rot_dim=16, vdim=32, kv_rank=48, q_rank=24, mlp="moe", expert_ff=64, experts=4)]
    cfg = oz.make_config(layers, width=64, loop=(1, 3, 2))
    W = oz.make_weights(cfg, seed=15, decay_rank=8)
    toks = prompt(cfg, 290, 32)
    want, mg = oracle(cfg, W, toks)
    llm = make_engine(kge, tmp_path, cfg, W, "bfloat16", bs=64)
    got = np.concatenate([run_pieces(llm, 0, toks[:150], [150]), run_pieces(llm, 0, toks[150:260], [3, 45, 2, 60]), run_pieces(llm, 0, toks[260:], [1] * 30)])
    llm.close()
    check(got, want, "bfloat16", "", mg, oz.bfloat16_noise(cfg, W, toks))


@pytest.mark.parametrize("shape", [(2, 32, 32, 64, True), (3, 96, 32, 128, False), (1, 64, 64, 128, True), (2, 16, 48, 64, False)])
def test_tensor_core_head_sizes(kge, tmp_path, shape):
    """bfloat16, 64-token pages, latent attention alone with keys and values of 64 or 128 numbers (unrotated + rotated
    part; values as wide as the keys): the sizes the tcgen05 prompt kernel and the TMA-staged decode kernels take.  Prompt
    steps, pieces, decoding over a page border, a decode batch of unequal contexts, single tokens beside a prompt piece."""
    heads, dim, rot_dim, vdim, gated = shape
    L = oz.latent_layer(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=24, q_rank=40, gated=gated, scale=1.6 / (dim + rot_dim) ** 0.5, mlp=None)
    cfg = oz.make_config([L], width=64, loop=(0, 1, 2))
    W = oz.make_weights(cfg, seed=23)
    toks = prompt(cfg, 230, 34)
    want = oz.forward(cfg, W, toks)
    noise = oz.bfloat16_noise(cfg, W, toks)
    llm = make_engine(kge, tmp_path, cfg, W, "bfloat16", bs=64, tokens=1024)
    check(run_pieces(llm, 0, toks, [230]), want, "bfloat16", "whole", None, noise)
    llm.trace_end(0)
    got = np.concatenate([run_pieces(llm, 1, toks[:180], [61, 3, 2, 64, 50]), run_pieces(llm, 1, toks[180:], [1] * 50)])
    check(got, want, "bfloat16", "pieces, then decoding", None, noise)
    # two requests decoding side by side (one far longer than the other) and a third that brings a prompt piece
    a, b = prompt(cfg, 150, 35), prompt(cfg, 9, 36)
    wa, wb = oz.forward(cfg, W, a).numpy(), oz.forward(cfg, W, b).numpy()
    llm.trace_add(2, a[:140])
    llm.trace_add(3, b[:3])
    llm.trace_step([(2, 140, []), (3, 3, [])])
    ga, gb = [], []
    for i in range(6):
        llm.trace_add(2, a[140 + i:141 + i])
        llm.trace_add(3, b[3 + i:4 + i])
        lg = llm.trace_step([(2, 1, [0]), (3, 1, [0])])
        ga.append(lg[0])
        gb.append(lg[1])
    c, d1 = prompt(cfg, 70, 37), prompt(cfg, 1, 38)
    llm.trace_end(3)
    llm.trace_add(2, a[146:147])
    llm.trace_add(4, c[:66])
    llm.trace_add(5, d1)
    lg = llm.trace_step([(2, 1, [0]), (4, 66, list(range(66))), (5, 1, [0])])
    llm.close()
    check(np.stack(ga), wa[140:146], "bfloat16", "long request of a decode batch", None, noise)
    check(np.stack(gb), wb[3:9], "bfloat16", "short request of a decode batch", None, noise)
    check(lg[:1], wa[146:147], "bfloat16", "a single token beside a prompt piece", None, noise)
    check(lg[1:67], oz.forward(cfg, W, c).numpy()[:66], "bfloat16", "a prompt piece beside single tokens", None, noise)
    check(lg[67:], oz.forward(cfg, W, d1).numpy(), "bfloat16", "a lone first token in a mixed step", None, noise)


def test_first_tokens(kge, tmp_path):
    cfg = full()
    W = oz.make_weights(cfg, seed=11)
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    for rid, n in enumerate([1, 2, 3, 5]):
        toks = prompt(cfg, n, 40 + n)
        got = run_pieces(llm, rid, toks, [n])
        llm.trace_end(rid)
        check(got, oz.forward(cfg, W, toks), "float32", f"{n} tokens")
    llm.close()


def test_long_decoding(kge, tmp_path):
    cfg = full()
    W = oz.make_weights(cfg, seed=12)
    toks = prompt(cfg, 200, 50)
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    got = run_pieces(llm, 0, toks, [4] + [1] * 196)
    llm.close()
    check(got, oz.forward(cfg, W, toks), "float32")


OTHER = [
    # one stream, no multiplier, one pass of the loop, a loop over everything
    dict(layers=[oz.latent_layer(heads=2, dim=5, rot_dim=2, vdim=3, kv_rank=4, q_rank=3, mlp="dense", ff=7, limit=0.9), oz.wkv_layer(heads=1, dim=7, mlp="moe", experts=2, top=1, expert_ff=5)],
         vocab=53, width=22, streams=1, residual_mult=1.0, loop=(0, 2, 1), eps=1e-3),
    dict(layers=[oz.wkv_layer(heads=3, dim=6, mlp=None), oz.latent_layer(gated=True, heads=5, dim=4, rot_dim=6, vdim=4, kv_rank=20, base=50.0, scale=0.9, mlp="moe", experts=9, top=5, expert_ff=11, router_scale=0.7)],
         vocab=67, width=42, streams=4, residual_mult=0.15, loop=(0, 2, 2)),
    # rows of 84 / 36 bytes: nothing is 16-byte aligned
    dict(layers=[oz.latent_layer(heads=3, dim=2, rot_dim=4, vdim=6, kv_rank=5, q_rank=7, mlp="moe", experts=3, top=2, expert_ff=64), oz.wkv_layer(heads=2, dim=9, mlp="dense", ff=64),
                 oz.latent_layer(gated=True, heads=1, dim=10, rot_dim=2, vdim=18, kv_rank=9, mlp=None)], vocab=72, width=18, streams=3, loop=(1, 2, 3)),
    # a recurrence head wider than a warp, equal sizes everywhere
    dict(layers=[oz.wkv_layer(heads=1, dim=40, mlp="dense", ff=40), oz.latent_layer(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=8, q_rank=8, mlp="moe", experts=4, top=4, expert_ff=8)],
         vocab=80, width=40, streams=2, residual_mult=2.0),
    # recurrence heads of 80 and 136 channels (token by token also in prompts), keys of 128 + 64 numbers with values of 128, only part of the rotated part turns
    dict(layers=[oz.wkv_layer(heads=1, dim=80, mlp=None), oz.latent_layer(heads=2, dim=128, rot_dim=64, vdim=128, kv_rank=24, q_rank=16, scale=0.07, rot_dims=40, mlp=None),
                 oz.wkv_layer(heads=1, dim=136, mlp=None)], vocab=90, width=48, streams=2),
]


@pytest.mark.parametrize("sizes", OTHER)
def test_other_sizes(kge, tmp_path, sizes):
    cfg = oz.make_config(**sizes)
    W = oz.make_weights(cfg, seed=13, decay_rank=5)
    toks = prompt(cfg, 50, 60)
    want, mg = oracle(cfg, W, toks)
    llm = make_engine(kge, tmp_path, cfg, W, "float32")
    check(run_pieces(llm, 0, toks, [50]), want, "float32", "whole")
    check(run_pieces(llm, 1, toks, [13, 2, 1, 1, 1, 32]), want, "float32", "pieces")
    llm.close()
    llm = make_engine(kge, tmp_path, cfg, W, "bfloat16", name="b")        # the same sizes through the 16-bit kernels and their fallbacks
    noise = oz.bfloat16_noise(cfg, W, toks)
    check(run_pieces(llm, 0, toks, [50]), want, "bfloat16", "whole, bfloat16", mg, noise)
    check(run_pieces(llm, 1, toks, [13, 2, 1, 1, 1, 32]), want, "bfloat16", "pieces, bfloat16", mg, noise)
    llm.close()


def test_checkpoint_without_stream_tensors(kge, tmp_path):
    """A one-stream checkpoint that leaves out the hyper-connection tensors and the per-column scales runs as the plain
    residual x <- x + m f(norm(x))."""
    cfg = oz.make_config([oz.wkv_layer(mlp="dense"), oz.latent_layer(mlp="moe")], streams=1, residual_mult=0.7)
    W = oz.make_weights(cfg, seed=18)
    for k in W:
        if ".hc" in k or k.split(".")[-1] in ("ls1", "ls2"):
            W[k] = torch.ones_like(W[k])
    toks = prompt(cfg, 30, 61)
    want = oz.forward(cfg, W, toks)
    bare = {k: v for k, v in W.items() if ".hc" not in k and k.split(".")[-1] not in ("ls1", "ls2")}
    llm = make_engine(kge, tmp_path, cfg, bare, "float32")
    check(run_pieces(llm, 0, toks, [17, 13]), want, "float32")
    llm.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_scheduler(kge, tmp_path, dtype):
    """LLM.generate: the continuous-batching scheduler cuts the prompts into 16-token steps, admits the third request
    when a slot frees up, samples greedily, and replays its decode steps as a CUDA graph."""
    cfg = full()
    W = oz.make_weights(cfg, seed=14)
    prompts = [prompt(cfg, n, 70 + n) for n in (37, 5, 21)]
    llm = make_engine(kge, tmp_path, cfg, W, dtype, seqs=2, batched=16)
    outs = llm.generate(prompts, kge.SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    assert llm.kernel_launches > 0
    llm.close()
    for p, o in zip(prompts, outs):
        got = o.outputs[0].token_ids
        assert len(got) == 12
        toks = list(p)
        for k, g in enumerate(got):       # teacher-forced: a different choice must be a near-tie of the oracle
            lg = oz.forward(cfg, W, toks)[-1]
            best = int(torch.argmax(lg))
            if g != best:      # the samplers read 16-bit logits rows: two logits within their spacing tie
                gap = float(lg[best] - lg[g])
                assert gap < (2.0 ** -7 * max(1.0, float(lg[best].abs())) if dtype == "float32" else 0.15), f"token {k}: chose {g}, oracle {best} leads by {gap}"
            toks.append(g)


def test_trace_runner_command_line(kge, tmp_path):
    """bin/trace_run end to end on this design: pieces of two requests side by side, a request that ends and one that
    takes its pages and slot, both number formats."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = oz.make_config([oz.wkv_layer(mlp="moe"), oz.latent_layer(gated=True, mlp="dense"), oz.latent_layer(mlp=None)], loop=(0, 2, 2))
    W = oz.make_weights(cfg, seed=17)
    d = str(tmp_path / "m")
    oz.save_model_dir(d, cfg, W)
    P = {"a": prompt(cfg, 50, 80), "b": prompt(cfg, 31, 81), "c": prompt(cfg, 40, 82)}
    want = {k: oz.forward(cfg, W, v).numpy() for k, v in P.items()}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": P["a"][:30], "want": [0, 29]}, {"id": "b", "tokens": P["b"][:2], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": P["b"][2:], "want": [0, 28]}, {"id": "a", "tokens": P["a"][30:31], "want": [0]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": P["a"][31:], "want": [18]}, {"id": "c", "tokens": P["c"], "want": [39, 5]}], "end": ["a", "c"]},
    ]
    rows = {0: [("a", 0), ("a", 29)], 1: [("b", 2), ("b", 30), ("a", 30)], 2: [("a", 49), ("c", 39), ("c", 5)]}
    for dtype in ("float32", "bfloat16"):
        out = str(tmp_path / ("out_" + dtype))
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", out, "--max-tokens", "128"],
                           input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        for st, rr in rows.items():
            got = np.fromfile(os.path.join(out, f"{st}.f32"), dtype="<f4").reshape(len(rr), cfg["vocab"])
            check(got, np.stack([want[k][i] for k, i in rr]), dtype, f"step {st}")


def test_server_command_line_and_sampling(kge, tmp_path):
    """`vllm serve DIR` picks the design from config.json: greedy completions over HTTP (token-id prompts) equal the
    in-process engine's, in bfloat16 and with --dtype float32; sampling with a temperature and a seed is reproducible and
    stays inside the vocabulary."""
    import json
    import os
    import socket
    import subprocess
    import time
    import urllib.request
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    binary = os.path.join(root, "kubernetes-gpu-cluster_b200", "bin", "vllm")
    assert os.path.exists(binary), "build the server: make -C kubernetes-gpu-cluster_b200"
    cfg = full()
    W = oz.make_weights(cfg, seed=19)
    d = str(tmp_path / "m")
    oz.save_model_dir(d, cfg, W)
    prompts = [prompt(cfg, n, 100 + n) for n in (23, 4, 40)]
    for dtype in ("bfloat16", "float32"):
        llm = kge.LLM(d, dtype=dtype, max_model_len=128, max_num_seqs=4, max_num_batched_tokens=32, num_gpu_blocks_override=16, enable_prefix_caching=False)
        ref = [o.outputs[0].token_ids for o in llm.generate(prompts, kge.SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))]
        warm = [o.outputs[0].token_ids for o in llm.generate(prompts[:1], kge.SamplingParams(max_tokens=8, temperature=0.8, top_k=20, seed=7, ignore_eos=True))]
        again = [o.outputs[0].token_ids for o in llm.generate(prompts[:1], kge.SamplingParams(max_tokens=8, temperature=0.8, top_k=20, seed=7, ignore_eos=True))]
        llm.close()
        assert warm == again and all(0 <= t < cfg["vocab"] for t in warm[0])
        s = socket.socket()
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
        s.close()
        proc = subprocess.Popen([binary, "serve", d, "--host", "127.0.0.1", "--port", str(port), "--dtype", dtype, "--max-model-len", "128", "--max-num-seqs", "4",
                                 "--max-num-batched-tokens", "32", "--num-gpu-blocks-override", "16", "--served-model-name", "z", "--trust-remote-code"],
                                stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
        try:
            t0 = time.time()
            while True:
                try:
                    with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                        if r.status == 200:
                            break
                except Exception:
                    pass
                assert proc.poll() is None, proc.stderr.read()[-2000:]
                assert time.time() - t0 < 120, "server did not come up"
                time.sleep(0.2)
            req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", headers={"Content-Type": "application/json"},
                                         data=json.dumps({"model": "z", "prompt": prompts, "max_tokens": 8, "temperature": 0, "ignore_eos": True}).encode())
            with urllib.request.urlopen(req, timeout=60) as r:
                body = json.loads(r.read().decode())
            assert [c["token_ids"] for c in body["choices"]] == ref, dtype
        finally:
            proc.terminate()
            try:
                proc.wait(timeout=20)
            except subprocess.TimeoutExpired:
                proc.kill()
