"""The Sagupel design in the engine against the plain implementation (``plain_sagupel``): every mechanism alone, whole
prompts against token-by-token decoding, portions down to two tokens, batches of unequal requests, slots and pages
that are used again, keys far away and at the edges of windows and pages, the first tokens, long decoding, sizes that
are 1 or equal, generation through the library's own loop, and trace replay (needs a B200)."""
import numpy as np
import pytest
import torch

import plain_sagupel as ps
import sagupel_helpers as sh
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


def f32(a):
    return np.float32(a).astype(np.float64)


class Step:
    """What the kernels read of a step: T packed tokens of sequences with these new and earlier lengths."""

    def __init__(self, new, before, slots=None):
        self.n_seqs, self.n_tokens = len(new), sum(new)
        self.single_token = all(n == 1 for n in new)
        cu = np.concatenate([[0], np.cumsum(new)])
        self.cu_seqlens = dev(cu, torch.int32)
        self.tok_seq = dev(np.repeat(np.arange(len(new)), new), torch.int32)
        self.tok_pos = dev(np.concatenate([np.arange(b, b + n) for n, b in zip(new, before)]), torch.int32)
        self.slots = dev(slots if slots is not None else np.arange(len(new)), torch.int32)


# ----------------------------------------------------------------------------- kernels alone
def test_norm_after_the_sum_clamped_gate_and_normed_embedding():
    rng = np.random.default_rng(1)
    for T, D in ((9, 100), (3, 256), (5, 4096 + 64)):
        x, y, w = f32(rng.standard_normal((T, D))), f32(rng.standard_normal((T, D))), f32(1 + 0.3 * rng.standard_normal(D))
        for alpha in (2.0, 1.0, 0.25):
            want = ps.rms_norm(alpha * x + y, w, EPS)
            for cast in (None, torch.float32, torch.bfloat16):
                h = dev(x)
                out = ops.rmsnorm_mix(h, dev(y), dev(w), EPS, alpha, cast)
                assert np.abs(h.double().cpu().numpy() - want).max() <= 1e-5
                assert (out is None) == (cast is None)
                if cast == torch.float32:
                    assert out is h
                if cast == torch.bfloat16:
                    assert np.array_equal(out.double().cpu().numpy(), h.to(torch.bfloat16).double().cpu().numpy())
    T = 9
    for F, inter in ((24, 0), (24, 8), (7, 0)):
        g, u = f32(3 * rng.standard_normal((T, F))), f32(3 * rng.standard_normal((T, F)))
        gu = np.concatenate([g, u], axis=1)
        if inter:
            gu = np.concatenate([np.concatenate([g[:, i:i + inter], u[:, i:i + inter]], axis=1) for i in range(0, F, inter)], axis=1)
        for limit in (1.5, 0.5, 7.0):
            got = ops.silu_mul(dev(gu), torch.float32, inter, "clamped_swish", limit).double().cpu().numpy()
            gc, uc = np.minimum(g, limit), np.clip(u, -limit, limit)
            assert np.abs(got - gc * ps.sigmoid(1.702 * gc) * (uc + 1.0)).max() <= 1e-5
        assert np.abs(ops.silu_mul(dev(gu), torch.float32, inter).double().cpu().numpy() - ps.silu(g) * u).max() <= 1e-5
    V, D = 31, 48
    table, nw = ps.round_bf16(rng.standard_normal((V, D))), f32(1 + 0.3 * rng.standard_normal(D))
    ids = rng.integers(0, V, 11)
    for tdtype in DTYPES:
        part = build_part("embedding", PartSpec("token", {"vocab_size": V, "hidden_size": D, "name": "embed", "norm": "embed.norm",
                                                          "norm_eps": EPS}), Runtime(DEV, tdtype))
        part.bind({"embed": dev(table, tdtype), "embed.norm": dev(nw)})
        assert np.abs(part.forward(dev(ids, torch.int32)).double().cpu().numpy() - ps.rms_norm(table[ids], nw, EPS)).max() <= 1e-5


@pytest.mark.parametrize("taps", [1, 2, 3, 5])
def test_input_convolution_whole_in_portions_and_token_by_token(taps):
    """x + conv(x) with its tail in slots that are not 0..B-1: unequal sequences whole, cut anywhere (also inside the taps'
    reach of the start), and token by token; bfloat16 output is the rounded 32-bit one."""
    rng = np.random.default_rng(taps)
    C, lens, slots = 40, [9, 1, 4], [5, 0, 3]
    xs = [f32(rng.standard_normal((n, C))) for n in lens]
    w = f32(0.6 * rng.standard_normal((C, taps)))
    refs = [ps.causal_conv(x, w, plus_input=True) for x in xs]
    for plan in ([lens], [[1, 1, 1], [2, 0, 3], [6, 0, 0]], [[1, 1, 1]] * 9):
        tail = torch.zeros((6, taps - 1, C), dtype=torch.float32, device=DEV)
        at, got = [0, 0, 0], [[], [], []]
        for counts in plan:
            who = [i for i, c in enumerate(counts) if c and at[i] < lens[i]]
            new = [min(counts[i], lens[i] - at[i]) for i in who]
            step = Step(new, [at[i] for i in who], [slots[i] for i in who])
            x = dev(np.concatenate([xs[i][at[i]:at[i] + n] for i, n in zip(who, new)]))
            out = ops.short_conv(x, 0, C, dev(w), None, tail, step, activation=False, plus_input=True).double().cpu().numpy()
            off = 0
            for i, n in zip(who, new):
                got[i].append(out[off:off + n])
                off += n
                at[i] += n
        for g, ref in zip(got, refs):
            assert np.abs(np.concatenate(g) - ref).max() <= 1e-5
    tail = torch.zeros((6, taps - 1, C), dtype=torch.float32, device=DEV)
    step = Step(lens, [0, 0, 0], slots)
    x = dev(np.concatenate(xs))
    a = ops.short_conv(x, 0, C, dev(w), None, tail.clone(), step, activation=False, plus_input=True)
    b = ops.short_conv(x, 0, C, dev(w), None, tail.clone(), step, activation=False, plus_input=True, out_dtype=torch.bfloat16)
    assert torch.equal(a.to(torch.bfloat16), b)


# ----------------------------------------------------------------------------- mixers alone
def make_mixer(entry, dtype, w, width, branch=None, taps=0):
    import questwend_b200  # noqa: F401
    from questwend_b200.config.registry import config_from_dict
    from questwend_b200.models.sagupel import _mixer
    cfg = config_from_dict(sh.config([(entry, None)], width=width, taps=taps))
    spec, pos_specs = _mixer(entry["type"], cfg.layers[0]["mixer"], width, EPS)
    if taps:
        spec = PartSpec("input_conv", {"inner": spec, "channels": width, "taps": taps, "weight": "l0.canon1"})
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


def plain_mixer(entry, x, w, dtype, branch=None, taps=0):
    r16 = dtype == torch.bfloat16
    m = entry["mixer"]
    if taps:
        x = ps.causal_conv(x, w["l0.canon1"], plus_input=True)
    if branch == 0:
        return ps.softmax_attention(x, m["left"], w, "l0.mix.left.", EPS, r16, biases=True, rotation=True, softcap=True, temp=True,
                                    talk=True, gate=True)
    if branch == 1:
        return ps.gated_delta(x, m["right"], w, "l0.mix.right.", EPS, r16)
    return ps.MIXERS[entry["type"]](x, m, w, "l0.mix.", EPS, r16)


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
    in_dtype = torch.float32 if part.reads_stream else dtype
    for counts in plan:
        who = [i for i, c in enumerate(counts) if c]
        chunks = [xs[i][at[i]:at[i] + counts[i]] for i in who]
        ctx = build_step_context(cache, [StepEntry(slots[i], [0] * counts[i], []) for i in who], 10 ** 6, DEV)[0]
        out = part.forward(dev(np.concatenate(chunks), in_dtype), ctx, unit).double().cpu().numpy()
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


RETENTIONS = [sh.retention(), sh.retention(heads=2, dim=24, vdim=40, dims=24, base=500.0, decay=(0.9, 0.999)),
              sh.retention(heads=1, dim=8, vdim=8, dims=None, decay=(1.0,)), sh.retention(heads=5, dim=12, vdim=5, dims=4),
              sh.retention(heads=2, dim=136, vdim=6, dims=64, decay=(0.5, 0.99)), sh.retention(heads=2, dim=64, vdim=64, dims=64)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("entry", RETENTIONS)
def test_retention_alone(entry, dtype):
    """Prompts of unequal lengths in one step (one crossing pages, one of a single token), then tokens one by one, then
    the same cut into portions."""
    width = 48
    w = sh.draw_weights(sh.config([(entry, None)], width=width), 6)
    rng = np.random.default_rng(7)
    lens, extra = [150, 4, 1], 9
    xs = [ps.round_bf16(rng.standard_normal((n + extra, width))) for n in lens]
    part = make_mixer(entry, dtype, w, width)
    refs = [plain_mixer(entry, x, w, dtype) for x in xs]
    for plan in (prompt_then_tokens(lens, extra), [[2, 2, 2], [100, 3, 1], [57, 8, 7]]):
        for g, ref in zip(run_mixer(part, dtype, xs, plan), refs):
            assert close(g, ref, dtype)


def test_retention_long_memory_in_portions_and_in_used_slots():
    """A decay close to 1 (the state remembers hundreds of tokens) and positions in the hundreds: whole, in portions and
    token by token, in slots whose state another sequence left behind."""
    entry, width, dtype = sh.retention(heads=2, dim=16, vdim=24, dims=16, base=100.0, decay=(0.999, 0.99)), 32, torch.float32
    w = sh.draw_weights(sh.config([(entry, None)], width=width), 4)
    x = ps.round_bf16(np.random.default_rng(5).standard_normal((500, width)))
    ref = plain_mixer(entry, x, w, dtype)
    assert np.abs(ref[-1] - plain_mixer(entry, x[250:], w, dtype)[-1]).max() > 100 * FP32_TOL * np.abs(ref).max()
    part = make_mixer(entry, dtype, w, width)
    cache = CacheManager([(part.kv_spec(), part.state_spec(), None)], 2048, 2, 600, dtype, DEV)
    for plan in ([[500]], [[257], [55], [188]], [[2]] * 250, [[440]] + [[1]] * 60):
        assert close(run_mixer(part, dtype, [x], plan, cache=cache)[0], ref, dtype), plan[0]


@pytest.mark.parametrize("entry", [sh.retention(heads=2, dim=16, vdim=24, dims=16, base=100.0, decay=(0.999, 0.99)),
                                   sh.retention(heads=3, dim=64, vdim=32, dims=32, decay=(1.0, 0.5, 0.96875)),
                                   sh.retention(heads=1, dim=128, vdim=128, dims=None, decay=(0.998,)),
                                   sh.retention(heads=2, dim=12, vdim=5, dims=4, decay=(0.0, 0.9))])
def test_retention_in_chunks_against_the_chain(entry):
    """Long prompts take the chunked form (chunks of 64 tokens side by side): unequal prompts that end inside a chunk, a
    portion that continues a state, and the state it leaves for the tokens after it, against the plain implementation and
    against the kernel that runs through the tokens one by one."""
    width, dtype = 32, torch.float32
    w = sh.draw_weights(sh.config([(entry, None)], width=width), 4)
    rng = np.random.default_rng(6)
    lens = [333, 130, 64]
    xs = [ps.round_bf16(rng.standard_normal((n + 5, width))) for n in lens]
    refs = [plain_mixer(entry, x, w, dtype) for x in xs]
    part = make_mixer(entry, dtype, w, width)
    for plan in ([lens] + [[1, 1, 1]] * 5, [[140, 1, 3], [193, 129, 61]] + [[1, 1, 1]] * 5):
        for g, ref in zip(run_mixer(part, dtype, xs, plan), refs):
            assert close(g, ref, dtype)
    saved = ops.RETENTION_CHUNKED_FROM
    try:
        ops.RETENTION_CHUNKED_FROM = 10 ** 9
        chain = run_mixer(part, dtype, xs, [lens] + [[1, 1, 1]] * 5)
    finally:
        ops.RETENTION_CHUNKED_FROM = saved
    for g, c, ref in zip(run_mixer(part, dtype, xs, [lens] + [[1, 1, 1]] * 5), chain, refs):
        assert np.abs(g - c).max() <= FP32_TOL * np.abs(ref).max()


LEFTS = [sh.left(), sh.left(heads=6, kv_heads=1, dim=8, dims=2, factor=0, scale=0.6, softcap=2.5),
         sh.left(heads=2, kv_heads=2, dim=64, dims=64, factor=8.0), sh.left(heads=3, kv_heads=3, dim=16, dims=None, softcap=0.0),
         sh.left(heads=2, kv_heads=1, dim=12, dims=4), sh.left(heads=1, kv_heads=1, dim=8, dims=8),
         sh.left(heads=8, kv_heads=4, dim=32, dims=16, scale=0.2), sh.left(heads=10, kv_heads=1, dim=136, dims=32, scale=0.1)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("left", LEFTS)
def test_mixed_heads_attention_alone(left, dtype):
    entry, width = sh.parallel(left, sh.right()), 48
    w = sh.draw_weights(sh.config([(entry, None)], width=width), 8, sharp=1.5)
    rng = np.random.default_rng(9)
    lens, extra = [150, 4, 1], 9
    xs = [ps.round_bf16(rng.standard_normal((n + extra, width))) for n in lens]
    part = make_mixer(entry, dtype, w, width, branch=0)
    refs = [plain_mixer(entry, x, w, dtype, branch=0) for x in xs]
    for plan in (prompt_then_tokens(lens, extra), [[2, 2, 2], [100, 3, 1], [57, 8, 7]]):
        for g, ref in zip(run_mixer(part, dtype, xs, plan), refs):
            assert close(g, ref, dtype)


RIGHTS = [sh.right(), sh.right(heads=3, kv_heads=3, dim=8, vdim=8, conv=2), sh.right(heads=1, kv_heads=1, dim=64, vdim=40, conv=1),
          sh.right(heads=4, kv_heads=2, dim=136, vdim=6, conv=3), sh.right(heads=6, kv_heads=1, dim=12, vdim=5, conv=5)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("right", RIGHTS)
def test_delta_rule_with_a_decay_per_head_alone(right, dtype):
    entry, width = sh.parallel(sh.left(), right), 48
    w = sh.draw_weights(sh.config([(entry, None)], width=width), 10)
    rng = np.random.default_rng(11)
    lens, extra = [150, 4, 1], 9
    xs = [ps.round_bf16(rng.standard_normal((n + extra, width))) for n in lens]
    part = make_mixer(entry, dtype, w, width, branch=1)
    refs = [plain_mixer(entry, x, w, dtype, branch=1) for x in xs]
    for plan in (prompt_then_tokens(lens, extra), [[2, 2, 2], [100, 3, 1], [57, 8, 7]]):
        for g, ref in zip(run_mixer(part, dtype, xs, plan), refs):
            assert close(g, ref, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_both_mixers_side_by_side_behind_the_input_convolution(dtype):
    entry, width = sh.MIXED["layers"][1], 64
    entry = {"type": entry["type"], "mixer": entry["mixer"]}
    w = sh.draw_weights(sh.config([(entry, None)], width=width, taps=3), 12)      # three taps here, four in the whole models
    rng = np.random.default_rng(13)
    lens, extra = [90, 3], 5
    xs = [f32(rng.standard_normal((n + extra, width))) for n in lens]
    part = make_mixer(entry, dtype, w, width, taps=3)
    assert len(part.state_spec()) == 3 and part.kv_spec().head_dim == 24 and part.reads_stream
    refs = [plain_mixer(entry, x, w, dtype, taps=3) for x in xs]
    for plan in (prompt_then_tokens(lens, extra), [[2, 2], [50, 1], [43, 5]]):
        for g, ref in zip(run_mixer(part, dtype, xs, plan), refs):
            assert close(g, ref, dtype)


WINDOWS = [sh.attention(), sh.attention(heads=6, kv_heads=2, dim=8, size=70), sh.attention(heads=3, kv_heads=3, dim=40, size=64, scale=0.2),
           sh.attention(heads=2, kv_heads=1, dim=12, size=5), sh.attention(heads=1, kv_heads=1, dim=8, size=1),
           sh.attention(heads=4, kv_heads=1, dim=80, size=150, scale=0.12), sh.attention(heads=2, kv_heads=2, dim=16, size=0),
           sh.attention(heads=12, kv_heads=1, dim=32, size=200, scale=0.2)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("entry", WINDOWS)
def test_window_attention_with_sink_and_slopes_alone(entry, dtype):
    width = 48
    w = sh.draw_weights(sh.config([(entry, None)], width=width), 14, sharp=1.5)
    rng = np.random.default_rng(15)
    lens, extra = [230, 4, 1], 9
    xs = [ps.round_bf16(rng.standard_normal((n + extra, width))) for n in lens]
    part = make_mixer(entry, dtype, w, width)
    refs = [plain_mixer(entry, x, w, dtype) for x in xs]
    for plan in (prompt_then_tokens(lens, extra), [[2, 2, 2], [100, 3, 1], [137, 8, 7]]):
        for g, ref in zip(run_mixer(part, dtype, xs, plan), refs):
            assert close(g, ref, dtype)


# ----------------------------------------------------------------------------- keys that stand out
def aligned(w, px, heads_per_key):
    """The key projection and norm made equal to the last query head's of every group (the head whose bias grows slowest
    with distance): a token's key then points where its own query points, and a query's weight goes to the tokens that
    repeat its own input (and to itself), far above every other key.  The values are the keys' raw projections, which
    differ from token to token in length."""
    dim = w[px + "q.norm"].shape[0]
    G = w[px + "k"].shape[0] // dim
    for g in range(G):
        head = g * heads_per_key + heads_per_key - 1
        w[px + "k"][g * dim:(g + 1) * dim] = w[px + "q"][head * dim:(head + 1) * dim]
        if px + "k.b" in w:
            w[px + "k.b"][g * dim:(g + 1) * dim] = w[px + "q.b"][head * dim:(head + 1) * dim]
    w[px + "k.norm"] = w[px + "q.norm"].copy()
    return w


def standing_out(T, width, seed, pairs):
    """Inputs in which, for each (query, keys) of ``pairs``, the keys' tokens repeat the query's direction at another
    length: with sharp q and k that query's weight goes to those keys if it sees them, and elsewhere if it does not."""
    x = np.random.default_rng(seed).standard_normal((T, width))
    for query, keys in pairs:
        for n, j in enumerate(keys):
            x[j] = x[query] * (1.5 + 0.5 * n)
    return ps.round_bf16(x)


@pytest.mark.parametrize("size", [20, 64, 70, 1, 130, 5])
def test_keys_at_the_edges_of_windows_and_pages(size):
    """A query's double sits at the window's first position (just inside), one before it (just outside), at the
    sequence's first positions, and at a page's first and last row: in a prompt, in a prompt cut there, and decoded.
    Sharp q and k: a key seen or missed by one position moves the output by far more than the tolerance."""
    entry, width, dtype = sh.attention(heads=2, kv_heads=1, dim=16, size=size, scale=0.5), 32, torch.float32
    w = aligned(sh.draw_weights(sh.config([(entry, None)], width=width), 8, sharp=3.0), "l0.mix.", 2)
    w["l0.mix.sink"] = np.array([2.0, -1.0])
    part = make_mixer(entry, dtype, w, width)
    for q in (4 * size + size // 2, 3 * size - 1, 3 * size, 129, 192, 2 * size + 1):
        T = q + 3
        first = q - size + 1
        cases = {"window_in": [first], "window_out": [first - 1], "first": [0], "second": [1],
                 "page_first": [64 * ((q - 1) // 64)], "page_last": [64 * ((q - 1) // 64) - 1], "before": [q - 1]}
        for name, keys in cases.items():
            keys = [j for j in keys if 0 <= j < q]
            if not keys:
                continue
            x = standing_out(T, width, q, [(q, keys)])
            ref = plain_mixer(entry, x, w, dtype)
            for plan in ([[T]], [[q], [3]], [[q], [1], [1], [1]], [[q - 1], [2], [2]]):
                if plan[0][0] <= 0:
                    continue
                assert close(run_mixer(part, dtype, [x], plan)[0], ref, dtype), (q, name, plan[0])
    if size >= 5:      # the sharpness does what the test needs: seeing the key or not changes the output by much more
        q = 2 * size + size // 2
        inside, outside = standing_out(q + 1, width, 1, [(q, [q - size + 1])]), standing_out(q + 1, width, 1, [(q, [q - size])])
        a, b = plain_mixer(entry, inside, w, dtype)[q], plain_mixer(entry, outside, w, dtype)[q]
        assert np.abs(a - b).max() > 100 * FP32_TOL * np.abs(a).max()


def test_a_far_key_among_hundreds_and_the_first_tokens():
    """700 tokens, causal attention with mixed heads: the query's only double is hundreds of positions back, at the first
    position, or at a page's edge; whole, cut, and decoded."""
    entry = sh.parallel(sh.left(heads=2, kv_heads=2, dim=16, dims=None, scale=0.5, softcap=50.0), sh.right())
    width, dtype, T = 32, torch.float32, 700
    w = aligned(sh.draw_weights(sh.config([(entry, None)], width=width), 9, sharp=3.0), "l0.mix.left.", 1)
    pairs = [(T - 1, [70]), (650, [127]), (300, [0]), (690, [1]), (500, [448]), (660, [63])]
    x = standing_out(T, width, 10, pairs)
    ref = plain_mixer(entry, x, w, dtype, branch=0)
    gone = x.copy()
    gone[70] = -gone[70]
    assert np.abs(ref[T - 1] - plain_mixer(entry, gone, w, dtype, branch=0)[T - 1]).max() > 100 * FP32_TOL * np.abs(ref).max()
    part = make_mixer(entry, dtype, w, width, branch=0)
    for plan in ([[T]], [[640]] + [[1]] * 60, [[299], [2], [399]]):
        assert close(run_mixer(part, dtype, [x], plan)[0], ref, dtype), plan[0]


def test_the_sink_takes_its_share():
    """A sink far above every score takes nearly all of the softmax's mass, one far below none: the plain implementation
    says so, and the engine agrees with it in both cases, in a prompt and decoded."""
    entry, width, dtype = sh.attention(heads=2, kv_heads=1, dim=16, size=40, scale=0.3), 32, torch.float32
    w = sh.draw_weights(sh.config([(entry, None)], width=width), 3)
    x = ps.round_bf16(np.random.default_rng(4).standard_normal((90, width)))
    outs = {}
    for name, sink in (("low", [-30.0, -30.0]), ("high", [30.0, 30.0]), ("mixed", [4.0, -2.0])):
        w["l0.mix.sink"] = np.array(sink)
        outs[name] = plain_mixer(entry, x, w, dtype)
        part = make_mixer(entry, dtype, w, width)
        for plan in ([[90]], [[80]] + [[1]] * 10):
            assert np.abs(run_mixer(part, dtype, [x], plan)[0] - outs[name]).max() <= FP32_TOL * np.abs(outs["low" if name == "high" else name]).max()
    assert np.abs(outs["high"]).max() < 1e-6 * np.abs(outs["low"]).max()


# ----------------------------------------------------------------------------- the prompt kernel on the tensor cores
TWO_PASS_FROM = ops.BIAS_TWO_PASS_FROM_KEYS


def shaped_oracle(q, k, v, pos0, scale, head_scale, softcap, slopes, window, sinks, mix, gate):
    """q [n, H, dim], k [L, G, dim], v [L, G, vdim] of one sequence (float64); the n queries sit at pos0 .. pos0 + n - 1.
    Returns [n, H * vdim]."""
    n, H, L, G = q.shape[0], q.shape[1], k.shape[0], k.shape[1]
    i, j = np.arange(pos0, pos0 + n)[:, None], np.arange(L)[None, :]
    seen = (j <= i) & ((i - j < window) if window > 0 else True)
    weights = np.zeros((H, n, L))
    for h in range(H):
        s = q[:, h] @ k[:, h // (H // G)].T * scale * (head_scale[h] if head_scale is not None else 1.0)
        if softcap > 0:
            s = softcap * np.tanh(s / softcap)
        if slopes is not None:
            s = s - slopes[h] * (i - j)
        s = np.where(seen, s, -np.inf)
        top = s.max(-1, keepdims=True)
        if sinks is not None:
            top = np.maximum(top, sinks[h])
        e = np.exp(s - top)
        weights[h] = e / (e.sum(-1, keepdims=True) + (np.exp(sinks[h] - top) if sinks is not None else 0.0))
    if mix is not None:
        weights = np.einsum("hg,gij->hij", mix, weights)
    out = np.stack([weights[h] @ v[:, h // (H // G)] for h in range(H)], axis=1)
    if gate is not None:
        out = out * ps.sigmoid(gate)[:, :, None]
    return out.reshape(n, -1)


@pytest.mark.parametrize("H, G, dim, vdim, window, extras", [
    (4, 2, 64, 64, 0, "cap temp mix gate"), (8, 4, 32, 32, 0, "mix"), (4, 1, 80, 80, 150, "slopes sink"), (2, 2, 16, 24, 70, "slopes sink cap"),
    (6, 2, 128, 128, 64, "sink"), (4, 2, 64, 64, 100, "slopes sink"), (8, 1, 128, 128, 0, "slopes"), (3, 1, 48, 8, 1, "slopes"), (2, 1, 256, 256, 0, "gate"), (5, 5, 16, 40, 200, "temp slopes sink mix gate cap")])
def test_prompt_kernels_and_the_decode_kernel_against_an_oracle(H, G, dim, vdim, window, extras):
    """Random queries and a random cache: unequal prompts whole and as later portions (queries that start at a position
    above 0, inside a page), and single tokens, on the tensor cores and on the plain kernels."""
    rng = np.random.default_rng(H * 1000 + dim)
    spec = __import__("questwend_b200.parts.base", fromlist=["KVSpec"]).KVSpec(G, dim, window, value_dim=vdim)
    lens, new = [300, 70, 17, 1], [[300, 70, 17, 1], [121, 70, 3, 1], [1, 1, 1, 1]]
    head_scale = f32(1 + 0.4 * rng.standard_normal(H)) if "temp" in extras else None
    slopes = f32([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)]) if "slopes" in extras else None
    sinks = f32(1 + rng.standard_normal(H)) if "sink" in extras else None
    mix = f32(np.eye(H) + 0.4 * rng.standard_normal((H, H))) if "mix" in extras else None
    softcap = 3.0 if "cap" in extras else 0.0
    for dtype in DTYPES:
        cache = CacheManager([(spec, None, None)], sum(lens) + 64 * 5, 4, 400, dtype, DEV)
        unit = cache.unit_cache(0)
        ks = [ps.round_bf16(rng.standard_normal((n, G, dim))) for n in lens]
        vs = [ps.round_bf16(rng.standard_normal((n, G, vdim))) for n in lens]
        for counts in new:
            slots = cache.open(4)
            before = [n - c for n, c in zip(lens, counts)]
            for s, n in zip(slots, before):
                if n:
                    build_step_context(cache, [StepEntry(s, [0] * n, [])], 10, DEV)
                    cache.advance(s, n)
            ctx = build_step_context(cache, [StepEntry(s, [0] * c, []) for s, c in zip(slots, counts)], 10, DEV)[0]
            table = ctx.page_tables[unit.group_id].cpu().numpy()
            for b, (k, v) in enumerate(zip(ks, vs)):                 # the cache as a prep kernel would have left it
                for p in range(lens[b]):
                    unit.k_pool[table[b, p // 64], :, p % 64] = dev(k[p], dtype)
                    unit.v_pool[table[b, p // 64], :, p % 64] = dev(v[p], dtype)
            qs = [ps.round_bf16(rng.standard_normal((c, H, dim))) for c in counts]
            gates = [f32(rng.standard_normal((c, H))) for c in counts] if "gate" in extras else None
            want = np.concatenate([shaped_oracle(q, k, v, n0, 0.3, head_scale, softcap, slopes, window, sinks, mix,
                                                 None if gates is None else gates[b])
                                   for b, (q, k, v, n0) in enumerate(zip(qs, ks, vs, before))])
            gate = None if gates is None else dev(np.concatenate([np.zeros((sum(counts), 3)), np.concatenate(gates)], axis=1))
            impls = ["auto", "two_pass"] if ctx.single_token else (["plain", "mma"] if dtype == torch.bfloat16 and dim % 16 == 0 else ["plain"])
            if (not ctx.single_token and dtype == torch.bfloat16 and dim == vdim and dim in (64, 128)
                    and not any(x in extras for x in ("temp", "cap", "mix", "gate"))):
                impls.append("tc")                                  # the tcgen05 kernel with the bias and the sink in its softmax
            for impl in impls:
                # single tokens with mixed heads: the form with all value heads, and the two passes over the keys
                ops.BIAS_TWO_PASS_FROM_KEYS = 0 if impl == "two_pass" else 10 ** 9
                impl = "auto" if impl == "two_pass" else impl
                got = ops.bias_attention(dev(np.concatenate(qs), dtype), unit.k_pool, unit.v_pool, ctx.page_tables[unit.group_id], ctx, 0.3,
                                         head_scale=None if head_scale is None else dev(head_scale), softcap=softcap,
                                         slopes=None if slopes is None else dev(slopes), window=window,
                                         sinks=None if sinks is None else dev(sinks), head_mix=None if mix is None else dev(mix),
                                         gate=gate, gate_col0=3, impl=impl).double().cpu().numpy()
                tol = 1e-4 if dtype == torch.float32 else 0.02
                assert np.abs(got - want).max() <= tol * max(np.abs(want).max(), 1.0), (dtype, counts, impl)
            cache.close(slots)
    ops.BIAS_TWO_PASS_FROM_KEYS = TWO_PASS_FROM


# ----------------------------------------------------------------------------- whole models
@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, cfgd, seed in (("mixed", sh.MIXED, 21), ("ones", sh.ONES, 22)):
        w = sh.draw_weights(cfgd, seed)
        out[name] = (sh.write_folder(str(tmp_path_factory.mktemp(name)), cfgd, w), cfgd, w)
    return out


def all_rows(eng, slot, tokens):
    return eng.step([StepEntry(slot, list(tokens), list(range(len(tokens))))]).double().cpu().numpy()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["mixed", "ones"])
def test_model_whole_in_batches_in_portions_and_decoded(models, which, dtype):
    folder, cfgd, w = models[which]
    td = torch.float32 if dtype == "float32" else torch.bfloat16
    eng = Engine.from_folder(folder, dtype=dtype, max_tokens=2048, max_batch=4)
    rng = np.random.default_rng(31)
    seqs = [rng.integers(0, cfgd["vocab"], n).tolist() for n in (150, 1, 7, 66)]
    refs = [ps.forward(cfgd, w, t, round16=td == torch.bfloat16) for t in seqs]
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
    """The stream after every layer against the plain implementation."""
    folder, cfgd, w = models["mixed"]
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_batch=2)
    tokens = np.random.default_rng(29).integers(0, cfgd["vocab"], 90).tolist()
    want = []
    ps.forward(cfgd, w, tokens, taps=want)
    (s,) = eng.open_sequences(1)
    ctx, rows = eng.build_context([StepEntry(s, tokens, [0])])
    got = []
    eng.model.forward(ctx, eng.unit_caches, rows, tap=lambda i, h: got.append(h.double().cpu().numpy()))
    assert len(got) == len(want) == 7
    for g, r in zip(got, want):
        assert np.abs(g - r).max() <= FP32_TOL * np.abs(r).max()


def test_long_decoding_over_windows_and_page_borders(models):
    folder, cfgd, w = models["mixed"]
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_batch=2)
    tokens = np.random.default_rng(19).integers(0, cfgd["vocab"], 280).tolist()
    ref = ps.forward(cfgd, w, tokens)
    (s,) = eng.open_sequences(1)
    rows = list(all_rows(eng, s, tokens[:2]))
    for t in tokens[2:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]).double().cpu().numpy()[0])
    assert close(np.stack(rows), ref, torch.float32)


def test_a_wide_model_with_many_rows(tmp_path):
    """Width 1,024 and a prompt of 600 tokens in bfloat16 (the sizes from which the products change kernels), then single
    tokens, and a batch of 20 single tokens."""
    cfgd = sh.config([(sh.retention(heads=4, dim=32, vdim=64, dims=16), sh.dense(ff=264)),
                      (sh.parallel(sh.left(heads=4, kv_heads=2, dim=32, dims=8), sh.right(heads=2, kv_heads=1, dim=32, vdim=64)), sh.dense(ff=72)),
                      (sh.attention(heads=4, kv_heads=1, dim=64, size=100, scale=0.12), sh.dense(ff=136))],
                     width=1024, vocab=128)
    w = sh.draw_weights(cfgd, 41)
    folder = sh.write_folder(str(tmp_path / "m"), cfgd, w)
    tokens = np.random.default_rng(3).integers(0, 128, 606).tolist()
    ref = ps.forward(cfgd, w, tokens, round16=True)
    eng = Engine.from_folder(folder, dtype="bfloat16", max_tokens=4096, max_batch=24)
    (s,) = eng.open_sequences(1)
    rows = list(all_rows(eng, s, tokens[:600]))
    for t in tokens[600:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]).double().cpu().numpy()[0])
    eng.close_sequences([s])
    assert close(np.stack(rows), ref, torch.bfloat16)
    slots = eng.open_sequences(20)
    out = eng.step([StepEntry(s, tokens[i:i + 3], [2]) for i, s in enumerate(slots)]).double().cpu().numpy()
    out2 = eng.step([StepEntry(s, [tokens[i + 3]], [0]) for i, s in enumerate(slots)]).double().cpu().numpy()
    for i in range(20):
        r = ps.forward(cfgd, w, tokens[i:i + 4], round16=True)
        assert close(out[i], r[2], torch.bfloat16) and close(out2[i], r[3], torch.bfloat16)


@pytest.mark.parametrize("layers", [[(sh.attention(heads=2, kv_heads=2, dim=8, size=6), sh.dense(ff=8))],
                                    [(sh.retention(heads=1, dim=8, vdim=8, dims=4), None)],
                                    [(sh.parallel(sh.left(heads=2, kv_heads=1, dim=8, dims=4), sh.right(heads=1, kv_heads=1, dim=8, vdim=8)), None)]],
                         ids=["no_state_but_the_tail", "one_state", "one_pair"])
def test_models_with_one_kind_of_mixer_only(layers, tmp_path):
    import questwend_b200 as qw
    cfgd = sh.config(layers, width=24, vocab=40, taps=2 if layers[0][1] else 0)
    w = sh.draw_weights(cfgd, 31)
    folder = sh.write_folder(str(tmp_path / "m"), cfgd, w)
    eng = Engine.from_folder(folder, dtype="float32", max_tokens=512, max_batch=3)
    tokens = np.random.default_rng(2).integers(0, 40, 70).tolist()
    ref = ps.forward(cfgd, w, tokens)
    (s,) = eng.open_sequences(1)
    rows = list(all_rows(eng, s, tokens[:66]))
    for t in tokens[66:]:
        rows.append(eng.step([StepEntry(s, [t], [0])]).double().cpu().numpy()[0])
    eng.close_sequences([s])
    assert close(np.stack(rows), ref, torch.float32)
    for use_graph in (True, False):
        out = qw.generate(eng, [tokens[:5], tokens[:1]], max_new_tokens=8, use_graph=use_graph)
        for p, r in zip([tokens[:5], tokens[:1]], out):
            full = ps.forward(cfgd, w, p + r.tokens)
            for j, tok in enumerate(r.tokens):
                row = full[len(p) - 1 + j]
                assert row.max() - row[tok] <= 2 * FP32_TOL * np.abs(full).max()


def test_generation_through_the_library_loop(models):
    """Greedy generation with the engine's own loop, scheduler, device sampler and CUDA graphs: two batches in slots that
    are used again, one request ending early, decoding across window edges and a page border; every chosen token is the
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
        assert stats.batches == 2 and res[2].finish_reason == "stop" and len(res[2].tokens) <= 7
        for run in (free, res):
            for p, r in zip(prompts, run):
                ref = ps.forward(cfgd, w, p + r.tokens)
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
    ra, rb = ps.forward(cfgd, w, a), ps.forward(cfgd, w, b)
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
    ref = ps.forward(cfgd, w, a + ids)
    for j, tok in enumerate(ids):
        row = ref[len(a) - 1 + j]
        assert row.max() - row[tok] <= 2 * FP32_TOL * np.abs(ref).max()
