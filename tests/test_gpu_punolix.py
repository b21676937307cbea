"""The Punolix design in the engine against the plain implementation (``plain_punolix``): every mechanism alone, whole
prompts against token-by-token decoding, portions down to two tokens, batches of unequal requests, slots and pages
that are used again, keys far away and at the edges of chunks and pages, the first tokens, long decoding, sizes that
are 1 or equal, generation through the library's own loop, and trace replay (needs a B200)."""
import numpy as np
import pytest
import torch

import plain_punolix as pp
import punolix_helpers as ph
from helpers import FP32_TOL, run_trace
from questwend_b200.cache import CacheManager
from questwend_b200.engine.engine import Engine, StepEntry, build_step_context
from questwend_b200.kernels import ops
from questwend_b200.parts import PartSpec, Runtime, build_part

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DTYPES = [torch.float32, torch.bfloat16]
BF16_RMS_TOL = 0.03         # bfloat16 engine against the plain implementation that rounds the products' operands, the
                            # queries and the cached keys and values: root mean square of the difference over the reference's
EPS = 1e-5


def close(got, ref, dtype, tol=FP32_TOL):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    if dtype == torch.float32:
        return np.abs(got - ref).max() <= tol * np.abs(ref).max()
    return np.sqrt(np.mean((got - ref) ** 2)) <= BF16_RMS_TOL * np.sqrt(np.mean(ref ** 2))


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dtype).to(DEV)


# ----------------------------------------------------------------------------- kernels alone
def test_stream_kernels_scaled_sum_reinjection_and_gated_gelu():
    rng = np.random.default_rng(1)
    T, D, V = 9, 100, 31
    x, y, w = rng.standard_normal((T, D)), rng.standard_normal((T, D)), 1 + 0.3 * rng.standard_normal(D)
    x32, y32, w32 = (np.float32(a).astype(np.float64) for a in (x, y, w))
    h = dev(x32)
    out = ops.rmsnorm(h, dev(w32), EPS, torch.float32, delta=dev(y32), write_sum=True, delta_scale=0.7).double().cpu().numpy()
    assert np.abs(h.double().cpu().numpy() - (x32 + 0.7 * y32)).max() <= 1e-6
    assert np.abs(out - pp.rms_norm(x32 + 0.7 * y32, w32, EPS)).max() <= 1e-5
    assert np.abs(ops.add_inplace(dev(x32), dev(y32), -1.5).double().cpu().numpy() - (x32 - 1.5 * y32)).max() <= 1e-6
    table, vec = pp.round_bf16(rng.standard_normal((V, D))), np.float32(rng.standard_normal(D)).astype(np.float64)
    ids = rng.integers(0, V, T)
    for tdtype in DTYPES:
        got = ops.embed_gather(dev(ids, torch.int32), dev(table, tdtype), scale=2.5).double().cpu().numpy()
        assert np.abs(got - 2.5 * table[ids]).max() <= 1e-6
        got = ops.embed_add(dev(x32), dev(ids, torch.int32), dev(table, tdtype), 2.5, dev(vec)).double().cpu().numpy()
        assert np.abs(got - (x32 + 2.5 * table[ids] + vec)).max() <= 1e-5
    assert np.abs(ops.embed_add(dev(x32), None, None, 1.0, dev(vec)).double().cpu().numpy() - (x32 + vec)).max() <= 1e-6
    for F, inter in ((24, 0), (24, 8), (7, 0)):
        g, u = np.float32(3 * rng.standard_normal((T, F))).astype(np.float64), np.float32(rng.standard_normal((T, F))).astype(np.float64)
        gu = np.concatenate([g, u], axis=1)
        if inter:
            gu = np.concatenate([np.concatenate([g[:, i:i + inter], u[:, i:i + inter]], axis=1) for i in range(0, F, inter)], axis=1)
        got = ops.silu_mul(dev(gu), torch.float32, inter, "gelu_tanh").double().cpu().numpy()
        assert np.abs(got - pp.gelu_tanh(g) * u).max() <= 1e-5
        assert np.abs(ops.silu_mul(dev(gu), torch.float32, inter).double().cpu().numpy() - pp.silu(g) * u).max() <= 1e-5


def test_wavelength_scaled_frequencies():
    from questwend_b200.parts.rotary import wavelength_scaled_frequencies
    for dims, base, sc in ((8, 10000.0, (4.0, 1.0, 4.0, 64)), (64, 5e5, (8.0, 1.0, 4.0, 8192)), (16, 100.0, (2.0, 0.5, 3.0, 20)), (2, 7.0, (3.0, 1.0, 2.0, 4))):
        ref = pp.frequencies(base, dims, dict(zip(("factor", "low", "high", "original"), sc)))
        got = wavelength_scaled_frequencies(dims, base, *sc).numpy()
        assert np.abs(got - ref).max() <= 1e-15 + 1e-12 * np.abs(ref).max()
        plain = pp.frequencies(base, dims)
        assert len({"kept" if a == b else "slowed" if abs(a - b / sc[0]) < 1e-15 else "between" for a, b in zip(ref, plain)}) >= (2 if dims > 2 else 1)


# ----------------------------------------------------------------------------- mixers alone
def make_mixer(entry, dtype, w, width, branch=None):
    import questwend_b200  # noqa: F401
    from questwend_b200.config.registry import config_from_dict
    from questwend_b200.models.punolix import _mixer
    cfg = config_from_dict(ph.config([(entry, None)], width=width)).with_tensor_shapes({k: v.shape for k, v in w.items()})
    spec, pos_specs = _mixer(entry["type"], cfg.layers[0]["mixer"], width, EPS)
    rt = Runtime(DEV, dtype)
    if isinstance(pos_specs, tuple):
        position = tuple(None if p is None else build_part("position", p, rt) for p in pos_specs)
    else:
        position = None if pos_specs is None else build_part("position", pos_specs, rt)
    part = build_part("mixer", PartSpec(spec.kind, spec.params, prefix="l0.mix."), rt, position=position)
    held = {}
    for t in part.tensors():
        assert tuple(w[t.name].shape) == tuple(t.shape), t.name
        held[t.name] = torch.from_numpy(w[t.name]).to(dtype if t.role == "matrix" else torch.float32).to(DEV)
    part.bind(held)
    return part if branch is None else part.branches[branch]


def plain_mixer(entry, x, w, dtype, branch=None):
    r16 = dtype == torch.bfloat16
    m = entry["mixer"]
    if branch == 0:
        return pp.chunked_attention(x, w, "l0.mix.left.", m["left"], EPS, r16)
    if branch == 1:
        return pp.gated_linear_attention(x, w, "l0.mix.right.", m["right"], EPS, r16)
    return pp.mixer(entry["type"], x, w, "l0.mix.", m, EPS, r16)


def run_mixer(part, dtype, xs, plan, cache=None):
    """``plan``: a list of steps, each a list of token counts per sequence (0: the sequence sits the step out).  Returns
    each sequence's outputs in order."""
    n_tokens = sum(len(x) for x in xs)
    if cache is None:
        cache = CacheManager([(part.kv_spec(), part.state_spec(), None)], n_tokens + 64 * len(xs) + 512, 8, max(len(x) for x in xs) + 64, dtype, DEV)
    unit = cache.unit_cache(0)
    slots = cache.open(len(xs))
    at = [0] * len(xs)
    got = [[] for _ in xs]
    for counts in plan:
        who = [i for i, c in enumerate(counts) if c]
        chunks = [xs[i][at[i]:at[i] + counts[i]] for i in who]
        ctx = build_step_context(cache, [StepEntry(slots[i], [0] * counts[i], []) for i in who], 10 ** 6, DEV)[0]
        out = part.forward(dev(np.concatenate(chunks), dtype), ctx, unit).double().cpu().numpy()
        off = 0
        for i, c in zip(who, chunks):
            got[i].append(out[off:off + len(c)])
            off += len(c)
            cache.advance(slots[i], len(c))
            at[i] += len(c)
    assert all(a == len(x) for a, x in zip(at, xs))
    cache.close(slots)
    return [np.concatenate(g) for g in got]


def prompt_then_tokens(lens, extra):
    return [list(lens)] + [[1] * len(lens)] * extra


DIFFERENTIALS = [ph.attention(), ph.attention(heads=3, kv_heads=3, dim=8, vdim=40, dims=8, base=500.0, softcap=2.5, diff=0.4),
                 ph.attention(heads=6, kv_heads=1, dim=8, vdim=8, dims=2, scale=0.6, softcap=0.0),
                 ph.attention(heads=2, kv_heads=2, dim=128, vdim=24, dims=64),
                 ph.attention(heads=2, kv_heads=1, dim=16, vdim=256, dims=0, diff=0.0),
                 ph.attention(heads=10, kv_heads=1, dim=8, vdim=16, dims=8),
                 ph.attention(heads=2, kv_heads=1, dim=12, vdim=20, dims=6),
                 ph.attention(heads=1, kv_heads=1, dim=8, vdim=8, dims=8, diff=0.7)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("entry", DIFFERENTIALS)
def test_differential_attention_alone(entry, dtype):
    """Prompts of unequal lengths in one step (one crossing pages, one of a single token), then tokens one by one."""
    width = 48
    w = ph.draw_weights(ph.config([(entry, None)], width=width), 6, sharp=1.5)
    rng = np.random.default_rng(7)
    lens, extra = [150, 4, 1], 9
    xs = [pp.round_bf16(rng.standard_normal((n + extra, width))) for n in lens]
    got = run_mixer(make_mixer(entry, dtype, w, width), dtype, xs, prompt_then_tokens(lens, extra))
    for g, x in zip(got, xs):
        assert close(g, plain_mixer(entry, x, w, dtype), dtype)


LEFTS = [ph.left(), ph.left(heads=6, kv_heads=1, dim=8, vdim=8, dims=2, conv=4, size=70, scale=0.6),
         ph.left(heads=2, kv_heads=2, dim=64, vdim=32, dims=64, conv=2, size=64, scaling=(8.0, 1.0, 4.0, 128)),
         ph.left(heads=3, kv_heads=3, dim=16, vdim=136, dims=0, conv=0, size=0),
         ph.left(heads=2, kv_heads=1, dim=12, vdim=20, dims=4, conv=3, size=5),
         ph.left(heads=1, kv_heads=1, dim=8, vdim=8, dims=8, conv=7, size=1),
         ph.left(heads=4, kv_heads=2, dim=32, vdim=16, dims=16, conv=3, size=200, scaling=(4.0, 1.0, 4.0, 64)),
         # keys and values of one size that the tcgen05 prompt kernel takes (bfloat16), chunks that cut its tiles
         ph.left(heads=4, kv_heads=2, dim=64, vdim=64, dims=32, conv=3, size=70, scale=0.2),
         ph.left(heads=3, kv_heads=1, dim=128, vdim=128, dims=128, conv=0, size=33, scale=0.15)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("left", LEFTS)
def test_chunked_attention_behind_its_convolution_alone(left, dtype):
    entry, width = ph.parallel(left, ph.right()), 48
    w = ph.draw_weights(ph.config([(entry, None)], width=width), 8, sharp=1.5)
    rng = np.random.default_rng(9)
    lens, extra = [150, 4, 1], 9
    xs = [pp.round_bf16(rng.standard_normal((n + extra, width))) for n in lens]
    part = make_mixer(entry, dtype, w, width, branch=0)
    refs = [plain_mixer(entry, x, w, dtype, branch=0) for x in xs]
    for plan in (prompt_then_tokens(lens, extra), [[2, 2, 2], [100, 3, 1], [57, 8, 7]]):
        for g, ref in zip(run_mixer(part, dtype, xs, plan), refs):
            assert close(g, ref, dtype)


RIGHTS = [ph.right(), ph.right(heads=3, dim=8, vdim=8, tau=3.0), ph.right(heads=1, dim=64, vdim=40, tau=16.0),
          ph.right(heads=2, dim=136, vdim=6, tau=1.0), ph.right(heads=5, dim=12, vdim=5, tau=2.0)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("right", RIGHTS)
def test_gated_linear_attention_alone(right, dtype):
    entry, width = ph.parallel(ph.left(), right), 48
    w = ph.draw_weights(ph.config([(entry, None)], width=width), 10, rank=7)
    rng = np.random.default_rng(11)
    lens, extra = [150, 4, 1], 9
    xs = [pp.round_bf16(rng.standard_normal((n + extra, width))) for n in lens]
    part = make_mixer(entry, dtype, w, width, branch=1)
    for g, x in zip(run_mixer(part, dtype, xs, prompt_then_tokens(lens, extra)), xs):
        assert close(g, plain_mixer(entry, x, w, dtype, branch=1), dtype)


def test_gated_linear_attention_long_memory_in_portions_and_token_by_token():
    """Decays close to 1 (the state remembers hundreds of tokens): whole, in portions and token by token, and in slots
    whose state another sequence left behind."""
    entry, width, dtype = ph.parallel(ph.left(), ph.right(heads=2, dim=16, vdim=24, tau=16.0)), 32, torch.float32
    w = ph.draw_weights(ph.config([(entry, None)], width=width), 4, slow_decay=True)
    x = pp.round_bf16(np.random.default_rng(5).standard_normal((500, width)))
    ref = plain_mixer(entry, x, w, dtype, branch=1)
    assert np.abs(ref[-1] - plain_mixer(entry, x[250:], w, dtype, branch=1)[-1]).max() > 100 * FP32_TOL * np.abs(ref).max()
    part = make_mixer(entry, dtype, w, width, branch=1)
    cache = CacheManager([(part.kv_spec(), part.state_spec(), None)], 2048, 2, 600, dtype, DEV)
    for plan in ([[500]], [[257], [55], [188]], [[2]] * 250, [[440]] + [[1]] * 60):
        assert close(run_mixer(part, dtype, [x], plan, cache=cache)[0], ref, dtype), plan[0]


@pytest.mark.parametrize("dtype", DTYPES)
def test_both_mixers_side_by_side(dtype):
    entry, width = ph.MIXED["layers"][1], 64
    entry = {"type": entry["type"], "mixer": entry["mixer"]}
    w = ph.draw_weights(ph.config([(entry, None)], width=width), 12)
    rng = np.random.default_rng(13)
    lens, extra = [90, 3], 5
    xs = [pp.round_bf16(rng.standard_normal((n + extra, width))) for n in lens]
    part = make_mixer(entry, dtype, w, width)
    assert len(part.state_spec()) == 2 and part.kv_spec().head_dim == 24
    for g, x in zip(run_mixer(part, dtype, xs, prompt_then_tokens(lens, extra)), xs):
        assert close(g, plain_mixer(entry, x, w, dtype), dtype)


# ----------------------------------------------------------------------------- keys that stand out
def aligned(w, px, n, conv):
    """The key projection (bias, taps, norm) made equal to the first query heads', and both made to read the first half of
    the input's coordinates only, the values the second half: a token's key then points where its own query points, and
    the query's weight goes to the tokens whose first half repeats its own (and to itself), far above every other key,
    while their values differ."""
    half = w[px + "q"].shape[1] // 2
    w[px + "q"][:, half:] = 0.0
    w[px + "v"][:, :half] = 0.0
    w[px + "k"], w[px + "k.b"] = w[px + "q"][:n].copy(), w[px + "q.b"][:n].copy()
    if conv:
        w[px + "k.conv"] = w[px + "q.conv"][:n].copy()
    if px + "k.norm" in w:
        w[px + "k.norm"] = w[px + "q.norm"].copy()
    return w


def standing_out(T, width, seed, pairs, span=1):
    """Inputs in which, for each (query, keys) of ``pairs``, the keys' tokens (and the ``span`` - 1 before each, which a
    convolution mixes in) repeat the first half of the query's: with sharp q and k that query's weight goes to those keys
    if it sees them, and elsewhere if it does not."""
    x = np.random.default_rng(seed).standard_normal((T, width))
    for query, keys in pairs:
        for j in keys:
            for back in range(span):
                if j - back >= 0 and query - back >= 0:
                    x[j - back, :width // 2] = x[query - back, :width // 2]
    return pp.round_bf16(x)


def turned_away(x, keys, span=1):
    """The same inputs with the keys of these tokens pointing the other way: what the query gives when it does not see them."""
    y = x.copy()
    for j in keys:
        y[max(j - span + 1, 0):j + 1, :x.shape[1] // 2] *= -1.0
    return y


@pytest.mark.parametrize("size, conv", [(20, 3), (64, 2), (70, 0), (1, 2), (130, 4), (5, 3)])
def test_keys_at_the_edges_of_chunks_and_pages(size, conv):
    """A query's double sits at the first position of the query's chunk (just inside), at the last of the chunk before
    (just outside), at the sequence's first position, and at a page's first and last row: in a prompt, in a prompt cut
    there, and decoded.  Sharp q and k: a key seen or missed by one position moves the output by far more than the
    tolerance."""
    left = ph.left(heads=2, kv_heads=1, dim=16, vdim=24, dims=0, conv=conv, size=size, scale=0.5)
    entry, width, dtype = ph.parallel(left, ph.right()), 32, torch.float32
    w = aligned(ph.draw_weights(ph.config([(entry, None)], width=width), 8, sharp=3.0), "l0.mix.left.", 16, conv)
    part = make_mixer(entry, dtype, w, width, branch=0)
    span = max(conv, 1)
    for q in (4 * size + size // 2, 3 * size - 1, 3 * size, 129, 192, 2 * size + 1):
        T = q + 3
        start = (q // size) * size
        cases = {"chunk_in": [start], "chunk_out": [start - 1], "first": [0], "second": [1],
                 "page_first": [64 * ((q - 1) // 64)], "page_last": [64 * ((q - 1) // 64) - 1], "before": [q - 1]}
        for name, keys in cases.items():
            keys = [j for j in keys if 0 <= j < q - span + 1]
            if not keys:
                continue
            x = standing_out(T, width, q, [(q, keys)], span)
            ref = plain_mixer(entry, x, w, dtype, branch=0)
            for plan in ([[T]], [[q], [3]], [[q], [1], [1], [1]], [[q - 1], [2], [2]]):
                if plan[0][0] <= 0:
                    continue
                assert close(run_mixer(part, dtype, [x], plan)[0], ref, dtype), (q, name, plan[0])
    if size >= 5:      # the sharpness does what the test needs: not seeing the key changes the output by much more
        q = 2 * size + size // 2
        x = standing_out(q + 1, width, 1, [(q, [2 * size])], span)
        a = plain_mixer(entry, x, w, dtype, branch=0)[q]
        b = plain_mixer(entry, turned_away(x, [2 * size], span), w, dtype, branch=0)[q]
        assert np.abs(a - b).max() > 100 * FP32_TOL * np.abs(a).max()


def test_a_far_key_among_hundreds_and_the_first_tokens():
    """700 tokens, causal differential attention: the query's only double is hundreds of positions back, at the first
    position, or at a page's edge; whole, cut, and decoded."""
    entry = ph.attention(heads=2, kv_heads=2, dim=16, vdim=16, dims=0, scale=0.5, softcap=50.0)
    width, dtype, T = 32, torch.float32, 700
    w = aligned(ph.draw_weights(ph.config([(entry, None)], width=width), 9, sharp=3.0), "l0.mix.", 64, 0)
    x = standing_out(T, width, 10, [(T - 1, [70]), (650, [127]), (300, [0]), (690, [1]), (500, [448]), (660, [63])])
    ref = plain_mixer(entry, x, w, dtype)
    assert np.abs(ref[T - 1] - plain_mixer(entry, turned_away(x, [70]), w, dtype)[T - 1]).max() > 100 * FP32_TOL * np.abs(ref).max()
    part = make_mixer(entry, dtype, w, width)
    for plan in ([[T]], [[640]] + [[1]] * 60, [[299], [2], [399]]):
        assert close(run_mixer(part, dtype, [x], plan)[0], ref, dtype), plan[0]


# ----------------------------------------------------------------------------- the prompt kernel on the tensor cores
def maps_oracle(q, k, v, pos0, maps, scale, softcap, chunk, lam, norm_out, eps, out_scale, H, G):
    """q [n, H, maps, dim], k [L, G, maps, dim], v [L, G, vdim] of one sequence (float64); the n queries sit at
    pos0 .. pos0 + n - 1.  Returns [n, H * vdim]."""
    n, L = q.shape[0], k.shape[0]
    out = np.zeros((n, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        maps_out = []
        for m in range(maps):
            s = q[:, h, m] @ k[:, g, m].T * scale
            if softcap > 0:
                s = softcap * np.tanh(s / softcap)
            i, j = np.arange(pos0, pos0 + n)[:, None], np.arange(L)[None, :]
            seen = (j <= i) & ((i // chunk == j // chunk) if chunk > 0 else True)
            s = np.where(seen, s, -np.inf)
            p = np.exp(s - s.max(axis=1, keepdims=True))
            maps_out.append((p / p.sum(axis=1, keepdims=True)) @ v[:, g])
        o = maps_out[0] - (lam * maps_out[1] if maps == 2 else 0.0)
        if norm_out:
            o = o / np.sqrt((o ** 2).mean(axis=1, keepdims=True) + eps) * out_scale
        out[:, h] = o
    return out.reshape(n, -1)


@pytest.mark.parametrize("maps, H, G, dim, vdim, chunk, softcap", [
    (2, 4, 2, 16, 32, 0, 3.0), (1, 6, 3, 32, 24, 70, 0.0), (2, 2, 1, 64, 128, 0, 0.0), (1, 2, 2, 128, 64, 64, 0.0),
    (1, 3, 1, 48, 8, 130, 2.0), (2, 2, 2, 32, 136, 200, 5.0), (1, 1, 1, 16, 16, 1, 0.0), (2, 8, 2, 16, 40, 5, 0.0),
    (1, 4, 2, 64, 64, 70, 0.0), (1, 8, 2, 128, 128, 200, 0.0), (1, 2, 2, 128, 128, 64, 0.0), (1, 6, 1, 64, 64, 0, 0.0),
    (1, 3, 3, 64, 64, 1, 0.0), (1, 16, 1, 128, 128, 33, 0.0)])
def test_tensor_core_prompt_kernel(maps, H, G, dim, vdim, chunk, softcap):
    """Sequences of unequal lengths with prompts that go on from cached tokens (positions that are not multiples of the
    tile), pages in a shuffled order; a key with a large score sits at the first position a query sees, at the one before
    it, at position 0 and at page borders.  Against float64 attention on the same bfloat16 inputs and against the plain
    kernel.  One uncapped map with keys and values of 64 or 128 also takes the tcgen05 kernel with its chunk mask."""
    from types import SimpleNamespace
    assert ops.maps_prefill_mma_fits(torch.bfloat16, maps, dim, vdim)
    tc = maps == 1 and softcap == 0.0 and dim == vdim and ops.tc_attention_fits(torch.bfloat16, dim, 64, H // G)
    rng = np.random.default_rng(dim + vdim + chunk)
    before, new = [0, 37, 200, 64, 5], [150, 91, 130, 1, 64]
    B, lam, eps, out_scale, scale = len(new), 0.35, 1e-5, 0.6, dim ** -0.5
    total = [a + b for a, b in zip(before, new)]
    width = max((t + 63) // 64 for t in total)
    order = rng.permutation(B * width + 3)
    table = np.zeros((B, width), dtype=np.int32)
    k_pool = torch.zeros((len(order), G, 64, maps * dim), dtype=torch.bfloat16, device=DEV)
    v_pool = torch.zeros((len(order), G, 64, vdim), dtype=torch.bfloat16, device=DEV)
    qs, ks, vs = [], [], []
    for b in range(B):
        L = total[b]
        k = pp.round_bf16(rng.standard_normal((L, G, maps, dim)))
        v = pp.round_bf16(rng.standard_normal((L, G, vdim)))
        q = pp.round_bf16(rng.standard_normal((new[b], H, maps, dim)))
        for i in range(0, new[b], 7):       # a key that stands out: at the edge of what query i sees, or just past it
            pos = before[b] + i
            first = (pos // chunk) * chunk if chunk > 0 else 0
            for j in (first, first - 1, 0, 64 * (pos // 64), 64 * (pos // 64) - 1)[i % 5:i % 5 + 1]:
                if 0 <= j < L:
                    k[j] = pp.round_bf16(3.0 * q[i, ::H // G] / np.sqrt(scale * dim))
        table[b, :(L + 63) // 64] = order[b * width:b * width + (L + 63) // 64]
        for page in range((L + 63) // 64):
            rows = slice(64 * page, min(64 * page + 64, L))
            k_pool[table[b, page], :, :rows.stop - rows.start] = dev(k[rows].reshape(-1, G, maps * dim).transpose(1, 0, 2), torch.bfloat16)
            v_pool[table[b, page], :, :rows.stop - rows.start] = dev(v[rows].transpose(1, 0, 2), torch.bfloat16)
        qs.append(q), ks.append(k), vs.append(v)
    cu = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    ctx = SimpleNamespace(single_token=False, n_seqs=B, max_new=max(new), max_len=max(total), cu_seqlens=dev(cu, torch.int32),
                          pos0=dev(np.array(before), torch.int32), seq_len=dev(np.array(total), torch.int32))
    q_all = dev(np.concatenate(qs).reshape(-1, H, maps * dim), torch.bfloat16)
    kw = dict(softcap=softcap, chunk=chunk, lam=lam, norm_out=maps == 2, eps=eps, out_scale=out_scale)
    gots = [ops.maps_attention(q_all, k_pool, v_pool, dev(table, torch.int32), ctx, maps, scale, impl=impl, **kw).double().cpu().numpy()
            for impl in (("mma", "tc") if tc else ("mma",))]
    if tc:
        ops.gemm_tc_check(DEV)
    plain = ops.maps_attention(q_all, k_pool, v_pool, dev(table, torch.int32), ctx, maps, scale, impl="plain", **kw).double().cpu().numpy()
    for b in range(B):
        ref = maps_oracle(qs[b], ks[b], vs[b], before[b], maps, scale, softcap, chunk, lam, maps == 2, eps, out_scale, H, G)
        rows = slice(cu[b], cu[b + 1])
        rms = np.sqrt(np.mean(ref ** 2))
        assert np.sqrt(np.mean((plain[rows] - ref) ** 2)) <= 0.006 * rms, b       # the output's own rounding to bfloat16
        for got in gots:
            assert np.sqrt(np.mean((got[rows] - ref) ** 2)) <= 0.012 * rms, b     # and the probabilities'
            assert np.abs(got[rows] - ref).max() <= 0.08 * np.abs(ref).max(), b


# ----------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfgd, seed in (("mixed", ph.MIXED, 11), ("ones", ph.ONES, 12)):
        w = ph.draw_weights(cfgd, seed)
        out[name] = (ph.write_folder(str(tmp_path_factory.mktemp(name)), cfgd, w), cfgd, w)
    return out


def all_rows(eng, slot, tokens):
    return eng.step([StepEntry(slot, tokens, list(range(len(tokens))))]).double().cpu().numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "ones"])
def test_whole_prompts_portions_batches_and_reuse(models, name, dtype):
    folder, cfgd, w = models[name]
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    V = cfgd["vocab"]
    rng = np.random.default_rng(13)
    seqs = [rng.integers(0, V, n).tolist() for n in (150, 1, 67, 9)]
    refs = [pp.forward(t, w, cfgd, td == torch.bfloat16) for t in seqs]
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=1024, max_batch=6)
    alone = []
    for t, ref in zip(seqs, refs):                          # each alone, whole
        (s,) = eng.open_sequences(1)
        alone.append(all_rows(eng, s, t))
        eng.close_sequences([s])
        assert close(alone[-1], ref, td)
    # all in one batch of unequal lengths, in slots and pages that were used before: the same as alone
    slots = eng.open_sequences(4)
    out = eng.step([StepEntry(s, t, list(range(len(t)))) for s, t in zip(slots, seqs)]).double().cpu().numpy()
    eng.close_sequences(slots)
    off = 0
    for t, ref, one in zip(seqs, refs, alone):
        assert close(out[off:off + len(t)], ref, td)
        if td == torch.float32:
            assert np.abs(out[off:off + len(t)] - one).max() <= FP32_TOL * np.abs(ref).max()
        off += len(t)
    # portions of several sizes, down to two tokens, in slots that were used before
    (s,) = eng.open_sequences(1)
    rows, at = [], 0
    for n in (2, 3, 60, 2, 17, 64, 2):
        rows.append(all_rows(eng, s, seqs[0][at:at + n]))
        at += n
    assert at == 150 and close(np.concatenate(rows), refs[0], td)
    eng.close_sequences([s])
    # prompts cut at unequal places, then token by token together; the shorter ones end earlier and give their slots back
    cuts = [60, 1, 3, 8]
    slots = eng.open_sequences(4)
    rows = {i: [] for i in range(4)}
    first = eng.step([StepEntry(s, t[:c], list(range(c))) for s, t, c in zip(slots, seqs, cuts)]).double().cpu().numpy()
    off = 0
    for i, c in enumerate(cuts):
        rows[i] += list(first[off:off + c])
        off += c
    pos, live = list(cuts), [i for i in range(4) if cuts[i] < len(seqs[i])]
    eng.close_sequences([slots[i] for i in range(4) if i not in live])
    while live:
        out = eng.step([StepEntry(slots[i], [seqs[i][pos[i]]], [0]) for i in live]).double().cpu().numpy()
        for r, i in enumerate(live):
            rows[i].append(out[r])
            pos[i] += 1
        done = [i for i in live if pos[i] == len(seqs[i])]
        eng.close_sequences([slots[i] for i in done])
        live = [i for i in live if i not in done]
    for i, ref in enumerate(refs):
        assert close(np.stack(rows[i]), ref, td), i
    assert eng.cache.slots.n_free == eng.max_batch and eng.cache.free_pages() == [g.pool.n for g in eng.cache._groups]


def test_layer_by_layer(models):
    """The stream after every scheduled run (a looped layer counts each time) against the plain implementation."""
    folder, cfgd, w = models["mixed"]
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_batch=2)
    tokens = np.random.default_rng(29).integers(0, cfgd["vocab"], 90).tolist()
    want = []
    pp.forward(tokens, w, cfgd, layers_out=want)
    (s,) = eng.open_sequences(1)
    ctx, rows = eng.build_context([StepEntry(s, tokens, [0])])
    got = []
    eng.model.forward(ctx, eng.unit_caches, rows, tap=lambda i, h: got.append(h.double().cpu().numpy()))
    assert len(got) == len(want) == 11
    for g, r in zip(got, want):
        assert np.abs(g - r).max() <= FP32_TOL * np.abs(r).max()


def test_long_decoding_over_chunks_and_page_borders(models):
    folder, cfgd, w = models["mixed"]
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_batch=2)
    tokens = np.random.default_rng(19).integers(0, cfgd["vocab"], 280).tolist()
    ref = pp.forward(tokens, w, cfgd)
    (s,) = eng.open_sequences(1)
    rows = list(all_rows(eng, s, tokens[:2]))
    for t in tokens[2:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]).double().cpu().numpy()[0])
    assert close(np.stack(rows), ref, torch.float32)


def test_a_wide_model_with_many_rows(tmp_path):
    """Width 2,048 and a prompt of 600 tokens in bfloat16 (the sizes from which the products change kernels), then single
    tokens."""
    cfgd = ph.config([(ph.attention(heads=4, kv_heads=2, dim=32, vdim=16, dims=8), ph.dense(ff=264)),
                      (ph.parallel(ph.left(heads=4, kv_heads=2, dim=32, vdim=16, dims=8, conv=3, size=100), ph.right()), ph.dense(ff=72))],
                     width=2048, vocab=128, loop=(0, 2, 2))
    w = ph.draw_weights(cfgd, 41)
    folder = ph.write_folder(str(tmp_path / "m"), cfgd, w)
    tokens = np.random.default_rng(3).integers(0, 128, 606).tolist()
    ref = pp.forward(tokens, w, cfgd, round16=True)
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=2048, max_batch=2)
    (s,) = eng.open_sequences(1)
    rows = list(all_rows(eng, s, tokens[:600]))
    for t in tokens[600:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]).double().cpu().numpy()[0])
    assert close(np.stack(rows), ref, torch.bfloat16)


def test_a_model_at_tensor_core_sizes_in_portions_and_batches(tmp_path):
    """bfloat16 with sizes that the tensor-core prompt kernels take (two maps of 32 with values of 64: both maps in one
    pass; one map of 64 with values of 64: the tcgen05 kernel with its chunk mask): a prompt whole, in portions that cut
    chunks and pages, and two unequal prompts in one batch against each alone, then single tokens."""
    cfgd = ph.config([(ph.attention(heads=4, kv_heads=2, dim=32, vdim=64, dims=16, softcap=4.0), ph.dense(ff=96)),
                      (ph.parallel(ph.left(heads=4, kv_heads=2, dim=64, vdim=64, dims=32, conv=3, size=70, scale=0.2),
                                   ph.right(heads=2, dim=16, vdim=24)), ph.dense(ff=72)),
                      (ph.attention(heads=2, kv_heads=1, dim=16, vdim=128, dims=16, softcap=0.0, diff=0.1), None)],
                     width=64, vocab=96, loop=(0, 2, 2))
    w = ph.draw_weights(cfgd, 43)
    folder = ph.write_folder(str(tmp_path / "m"), cfgd, w)
    rng = np.random.default_rng(5)
    long, short = rng.integers(0, 96, 330).tolist(), rng.integers(0, 96, 90).tolist()
    ref_long, ref_short = pp.forward(long, w, cfgd, round16=True), pp.forward(short, w, cfgd, round16=True)
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=2048, max_batch=3)
    for cuts in ([324], [139, 141, 44], [64, 70, 190]):
        (s,) = eng.open_sequences(1)
        rows, at = [], 0
        for n in cuts:
            rows += list(all_rows(eng, s, long[at:at + n]))
            at += n
        for t in long[at:]:
            rows.append(eng.step([StepEntry(s, [t], [0])]).double().cpu().numpy()[0])
        eng.close_sequences([s])
        assert close(np.stack(rows), ref_long, torch.bfloat16), cuts
    a, b = eng.open_sequences(2)
    out = eng.step([StepEntry(a, long[:324], list(range(324))), StepEntry(b, short[:84], list(range(84)))]).double().cpu().numpy()
    rows_a, rows_b = list(out[:324]), list(out[324:])
    for i in range(6):
        out = eng.step([StepEntry(a, [long[324 + i]], [0]), StepEntry(b, [short[84 + i]], [0])]).double().cpu().numpy()
        rows_a.append(out[0]), rows_b.append(out[1])
    assert close(np.stack(rows_a), ref_long, torch.bfloat16) and close(np.stack(rows_b), ref_short, torch.bfloat16)


@pytest.mark.parametrize("layers", [[(ph.attention(heads=2, kv_heads=2, dim=8, vdim=8, dims=8), ph.dense(ff=8))],
                                    [(ph.parallel(ph.left(heads=2, kv_heads=1, dim=8, vdim=8, dims=4, conv=2, size=6), ph.right(heads=1, dim=8, vdim=8)), None)]],
                         ids=["no_state", "one_pair"])
def test_models_with_one_kind_of_mixer_only(layers, tmp_path):
    import questwend_b200 as qw
    cfgd = ph.config(layers, width=24, vocab=40)
    w = ph.draw_weights(cfgd, 31)
    folder = ph.write_folder(str(tmp_path / "m"), cfgd, w)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_batch=3)
    tokens = np.random.default_rng(2).integers(0, 40, 70).tolist()
    ref = pp.forward(tokens, w, cfgd)
    (s,) = eng.open_sequences(1)
    rows = list(all_rows(eng, s, tokens[:66]))
    for t in tokens[66:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]).double().cpu().numpy()[0])
    eng.close_sequences([s])
    assert close(np.stack(rows), ref, torch.float32)
    for use_graph in (True, False):
        out = qw.generate(eng, [tokens[:5], tokens[:1]], max_new_tokens=8, use_graph=use_graph)
        for p, r in zip([tokens[:5], tokens[:1]], out):
            full = pp.forward(p + r.tokens, w, cfgd)
            for j, tok in enumerate(r.tokens):
                row = full[len(p) - 1 + j]
                assert row.max() - row[tok] <= 2 * FP32_TOL * np.abs(full).max()


def test_generation_through_the_library_loop(models):
    """Greedy generation with the engine's own loop, scheduler, device sampler and CUDA graphs: two batches in slots that
    are used again, one request ending early, decoding across chunk edges and a page border; every chosen token is the
    plain implementation's choice."""
    import questwend_b200 as qw
    folder, cfgd, w = models["mixed"]
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=1024, max_batch=3)
    rng = np.random.default_rng(17)
    prompts = [rng.integers(0, cfgd["vocab"], n).tolist() for n in (20, 1, 58, 5)]
    n_new = 24
    for use_graph in (True, False):
        free = qw.generate(eng, prompts, max_new_tokens=n_new, use_graph=use_graph)
        stop = free[2].tokens[6]
        stats = qw.GenerationStats()
        res = qw.generate(eng, prompts, max_new_tokens=n_new, stop_ids=[stop], use_graph=use_graph, stats=stats)
        assert stats.batches == 2 and res[2].finish_reason == "stop" and len(res[2].tokens) <= 6
        for run in (free, res):
            for p, r in zip(prompts, run):
                ref = pp.forward(p + r.tokens, w, cfgd)
                scale = np.abs(ref).max()
                for j, tok in enumerate(r.tokens):
                    row = ref[len(p) - 1 + j]
                    assert row.max() - row[tok] <= 2 * FP32_TOL * scale, (len(p), j, tok, int(row.argmax()))
    assert eng.cache.slots.n_free == eng.max_batch


def test_trace_replay_and_command_line(models, tmp_path):
    folder, cfgd, w = models["ones"]
    V = cfgd["vocab"]
    rng = np.random.default_rng(23)
    a, b = rng.integers(0, V, 9).tolist(), rng.integers(0, V, 4).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:7], "want": [0, 6]}, {"id": "b", "tokens": b[:3], "want": [2]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[7:8], "want": []}, {"id": "b", "tokens": b[3:], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[8:], "want": [0]}], "end": ["a"]}]
    out = run_trace(folder, "float32", steps, 256, str(tmp_path / "out"))
    ra, rb = pp.forward(a, w, cfgd), pp.forward(b, w, cfgd)
    assert close(out[0], np.stack([ra[0], ra[6], rb[2]]), torch.float32)
    assert close(out[1], rb[3:4], torch.float32) and close(out[2], ra[8:9], torch.float32)
    import os
    import subprocess
    import sys
    from helpers import ROOT
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qw-cli"), "-m", folder, "-p", " ".join(map(str, a)),
                           "-n", "5", "--dtype", "float32", "--n-ctx", "128"], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr
    ids = [int(x) for x in proc.stdout.split()]
    ref = pp.forward(a + ids, w, cfgd)
    for j, tok in enumerate(ids):
        row = ref[len(a) - 1 + j]
        assert row.max() - row[tok] <= 2 * FP32_TOL * np.abs(ref).max()
