"""Tracer / lowering tests (CPU): the expression graph recorded from a mod must evaluate
to what the Python mod itself returns on numpy arrays, the symbolic derivative must match
a finite difference, and the generated CUDA text must compile for sm_100a."""
import numpy as np
import pytest

from flaxattention_b200 import _cabi, fnp, modtrace
from flaxattention_b200.blockmask import and_masks, or_masks, noop_mask
from flaxattention_b200.masks import (causal_mask, generate_attention_sink, generate_causal_offset,
                                      generate_sliding_window)
from flaxattention_b200.mods import checkerboard, generate_alibi_bias


def _grid(B=2, H=3, Q=17, KV=19):
    b = np.arange(B, dtype=np.int32).reshape(B, 1, 1, 1)
    h = np.arange(H, dtype=np.int32).reshape(1, H, 1, 1)
    q = np.arange(Q, dtype=np.int32).reshape(1, 1, Q, 1)
    kv = np.arange(KV, dtype=np.int32).reshape(1, 1, 1, KV)
    s = np.random.default_rng(0).standard_normal((B, H, Q, KV)).astype(np.float32)
    return s, b, h, q, kv


def tanh_softcap(score, b, h, q, kv):
    return 30.0 * fnp.tanh(score / 30.0)


def rel_bias(score, b, h, q, kv):
    return score + fnp.abs(q - kv) * -0.25 + fnp.where(kv % 3 == 0, 1.0, 0.0) * (b + 1)


def floor_mix(score, b, h, q, kv):
    return score * fnp.exp2(-((q // 4) - (kv // 4)) / 8.0) + fnp.minimum(score, 0.5) - fnp.maximum(score, -0.5)


def neg_mod(score, b, h, q, kv):
    return fnp.where((q - kv) % -3 == -1, score * score, fnp.sigmoid(score))


SCORE_MODS = [generate_alibi_bias(8), checkerboard, tanh_softcap, rel_bias, floor_mix, neg_mod]
MASK_MODS = [causal_mask, generate_sliding_window(5), generate_attention_sink(6, 2), generate_causal_offset(3),
             and_masks(causal_mask, lambda b, h, q, kv: (kv + h) % 2 == 0),
             or_masks(lambda b, h, q, kv: kv < 2, lambda b, h, q, kv: ~(q < kv) & (b == 1)), noop_mask]


@pytest.mark.parametrize("fn", SCORE_MODS)
def test_score_mod_graph_matches_python(fn):
    s, b, h, q, kv = _grid()
    tm = modtrace.trace_score_mod(fn)
    got = modtrace.evaluate(tm, s, b, h, q, kv)
    want = np.asarray(fn(s, b, h, q, kv), dtype=np.float32)
    np.testing.assert_allclose(np.broadcast_to(got, want.shape), want, rtol=2e-6, atol=2e-6)


@pytest.mark.parametrize("fn", MASK_MODS)
def test_mask_mod_graph_matches_python(fn):
    s, b, h, q, kv = _grid()
    tm = modtrace.trace_mask_mod(fn)
    got = np.broadcast_to(modtrace.evaluate(tm, None, b, h, q, kv), s.shape)
    want = np.broadcast_to(np.asarray(fn(b, h, q, kv)).astype(bool), s.shape)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("fn", SCORE_MODS)
def test_symbolic_derivative(fn):
    s, b, h, q, kv = _grid()
    s = s.astype(np.float64)
    tm = modtrace.trace_score_mod(fn)
    g = modtrace.evaluate(modtrace.derivative(tm), s.astype(np.float32), b, h, q, kv)
    eps = 1e-3
    f = lambda x: np.asarray(fn(x, b, h, q, kv), dtype=np.float64)  # noqa: E731
    fd = (f(s + eps) - f(s - eps)) / (2 * eps)
    # exclude the kinks of min/max
    ok = (np.abs(np.abs(s) - 0.5) > 2 * eps)
    np.testing.assert_allclose(np.broadcast_to(g, fd.shape)[ok], fd[ok], rtol=2e-3, atol=2e-3)


def test_derivative_of_a_float_remainder():
    """score % c is score minus a step function: its derivative is 1 away from the steps
    (an integer remainder stays piecewise constant, derivative 0)."""
    def wrap(score, b, h, q, kv):
        return (score * 2.0) % 0.75 + ((q - kv) % 3) * 0.5

    s, b, h, q, kv = _grid()
    g = modtrace.evaluate(modtrace.derivative(modtrace.trace_score_mod(wrap)), s, b, h, q, kv)
    np.testing.assert_allclose(np.broadcast_to(g, s.shape), np.full(s.shape, 2.0, np.float32))


def test_python_mod_semantics():
    def m(score, b, h, q, kv):
        return fnp.where(((q - kv) % 4 == 3) & ((q - kv) // 4 == -1), 1.0, 0.0)

    s, b, h, q, kv = _grid()
    got = modtrace.evaluate(modtrace.trace_score_mod(m), s, b, h, q, kv)
    d = (q - kv)
    want = ((np.remainder(d, 4) == 3) & (np.floor_divide(d, 4) == -1)).astype(np.float32)
    assert np.array_equal(np.broadcast_to(got, want.shape), np.broadcast_to(want, want.shape))


def test_score_mod_as_mask():
    def neginf_future(score, b, h, q, kv):
        return fnp.where(q >= kv, score, -fnp.inf)

    s, b, h, q, kv = _grid()
    tm = modtrace.trace_mask_mod(neginf_future)
    got = np.broadcast_to(modtrace.evaluate(tm, None, b, h, q, kv), s.shape)
    assert np.array_equal(got, np.broadcast_to(q >= kv, s.shape))


def test_numpy_and_torch_function_interop():
    import torch

    def m_np(score, b, h, q, kv):
        return np.where(np.greater_equal(q, kv), np.exp2(score), np.tanh(score))

    def m_torch(score, b, h, q, kv):
        return torch.where(q >= kv, torch.exp2(score), torch.tanh(score))

    a = modtrace.to_cuda(modtrace.trace_score_mod(m_np), "f")
    c = modtrace.to_cuda(modtrace.trace_score_mod(m_torch), "f")
    assert a == c


def test_data_dependent_branch_is_rejected():
    def bad(score, b, h, q, kv):
        return score if q >= kv else -score

    with pytest.raises(TypeError):
        modtrace.trace_score_mod(bad)


def test_identity_and_noop_are_elided():
    ms = modtrace.lower_mods(lambda s, b, h, q, kv: s, noop_mask)
    assert "FA_HAS_SCORE_MOD 0" in ms.source and "FA_HAS_MASK_MOD 0" in ms.source
    ms2 = modtrace.lower_mods(checkerboard, causal_mask)
    assert ms2.key != ms.key and "FA_HAS_SCORE_MOD 1" in ms2.source


def test_lowered_mods_compile_for_sm100a(tmp_path):
    """Run-time compilation needs no GPU; every kernel kind must build with a real mod."""
    L = _cabi.lib()
    L.fa_set_cache_dir(str(tmp_path).encode())
    try:
        ms = modtrace.lower_mods(floor_mix, generate_attention_sink(64, 4))
        m = _cabi.Module(ms.source)
        before = L.fa_compile_count()
        m.prepare(_cabi.KIND_BLOCKMASK, 0, 64, 64)
        m.prepare(_cabi.KIND_FWD, _cabi.FA_BF16, 64, 64)
        after = L.fa_compile_count()
        assert after >= before + 2
        # a second module with the same source hits the on-disk cache
        m2 = _cabi.Module(ms.source)
        m2.prepare(_cabi.KIND_FWD, _cabi.FA_BF16, 64, 64)
        assert L.fa_compile_count() == after
        bad = _cabi.Module("#define FA_HAS_SCORE_MOD 1\n#define FA_HAS_MASK_MOD 0\nthis is not CUDA\n")
        with pytest.raises(_cabi.FlaxAttnError) as ei:
            bad.prepare(_cabi.KIND_FWD, _cabi.FA_F16, 64, 64)
        assert ei.value.code == -2
    finally:
        import os
        L.fa_set_cache_dir(os.path.join(os.path.dirname(_cabi.LIB_PATH), "_kernel_cache").encode())


def test_captured_buffers_trace_evaluate_and_lower():
    """Tensors a mod closes over and indexes with traced values become load nodes (the
    reference's score_mod_other_buffers, flaxattention/core/attention.py:22-23): numbered per
    mod pair, linear index from the strides, clamped in the generated code."""
    import torch

    doc = torch.tensor([0, 0, 0, 1, 1, 2, 2, 2, 2, 3], dtype=torch.int64)
    bias = torch.arange(4 * 10 * 10, dtype=torch.float32).reshape(4, 10, 10).transpose(1, 2)  # non-contiguous view

    def doc_mask(b, h, q, kv):
        return (doc[q] == doc[kv]) & (q >= kv)

    def bias_mod(s, b, h, q, kv):
        return s + bias[h, q, kv] * 2.0

    mt = modtrace
    ms = mt.lower_mods(bias_mod, doc_mask)
    assert len(ms.buffers) == 2 and ms.buffers[0] is bias and ms.buffers[1] is doc
    assert "FA_NUM_MOD_BUFS 2" in ms.source and "fa_ld_i64(1," in ms.source and "fa_ld_f32(0," in ms.source
    assert ms.affine is not None                      # score + table[...] is affine in the score
    q = np.arange(10)[:, None]
    kv = np.arange(10)[None, :]
    got = mt.evaluate(ms.mask, None, 0, 0, q, kv)
    assert np.array_equal(got, (doc.numpy()[q] == doc.numpy()[kv]) & (q >= kv))
    sc = np.linspace(-1, 1, 100, dtype=np.float32).reshape(10, 10)
    got = mt.evaluate(ms.score, sc, 0, 3, q, kv)
    assert np.allclose(got, sc + bias.numpy()[3][q, kv] * 2.0)
    assert np.all(mt.evaluate(ms.grad, sc, 0, 3, q, kv) == 1.0)
    # out-of-range indices (padding rows of a ragged tile) read a clamped element instead of faulting
    assert mt.evaluate(ms.mask, None, 0, 0, np.array([50]), np.array([9]))[0] == True  # noqa: E712  doc[9] == doc[clamp(50)]

    with pytest.raises(TypeError, match="2 dimensions"):
        mt.lower_mods(None, lambda b, h, q, kv: torch.zeros(3, 3)[q] > 0)
    with pytest.raises(TypeError, match="dtype"):
        mt.lower_mods(None, lambda b, h, q, kv: torch.zeros(3, dtype=torch.float16)[q] > 0)


def test_jaxpr_replay_builds_the_same_graph_as_the_tracer():
    """The jaxpr front end (for mods written with jax.numpy) replays a flat list of primitive
    applications on the tracer's symbols.  JAX is not needed to check the replay itself: the list
    below is what jax.make_jaxpr gives for the reference's ALiBi bias
    (score + (q - kv) * exp2(-(h + 1) * 8 / H), flaxattention/mods/alibi.py:15-18) and for a causal
    sliding window, written out by hand with stand-in equation objects."""
    from types import SimpleNamespace as NS

    from flaxattention_b200 import jax_frontend as jf

    class Var:
        pass

    def lit(v):
        return NS(val=v)

    def eqn(name, ins, outs, **params):
        return NS(primitive=NS(name=name), invars=ins, outvars=outs, params=params)

    s_, b_, h_, q_, kv_ = (Var() for _ in range(5))
    t = [Var() for _ in range(8)]
    alibi_eqns = [
        eqn("add", [h_, lit(1)], [t[0]]),
        eqn("convert_element_type", [t[0]], [t[1]], new_dtype=np.float32, weak_type=False),
        eqn("mul", [t[1], lit(-1.0)], [t[2]]),                       # -(h + 1) * 8 / 8
        eqn("pjit", [t[2]], [t[3]], jaxpr=NS(jaxpr=NS(constvars=[], invars=[t[2]], outvars=[t[6]],
                                                      eqns=[eqn("exp2", [t[2]], [t[6]])]), consts=[])),
        eqn("sub", [q_, kv_], [t[4]]),
        eqn("convert_element_type", [t[4]], [t[5]], new_dtype=np.float32, weak_type=False),
        eqn("mul", [t[5], t[3]], [t[7]]),
    ]
    out = Var()
    alibi_eqns.append(eqn("add", [s_, t[7]], [out]))
    jaxpr = NS(constvars=[], invars=[s_, b_, h_, q_, kv_], outvars=[out], eqns=alibi_eqns)

    def run():
        leaves = modtrace._leaf_syms()
        (res,) = jf._run_jaxpr(jaxpr, [], list(leaves))
        return modtrace.cast(modtrace._lift(res), modtrace.F32)

    tm = modtrace._traced(None, run, "score")
    s, b, h, q, kv = _grid(H=8)
    got = modtrace.evaluate(tm, s, b, h, q, kv)
    want = np.asarray(generate_alibi_bias(8)(s, b, h, q, kv), dtype=np.float32)
    np.testing.assert_allclose(np.broadcast_to(got, want.shape), want, rtol=2e-6, atol=2e-6)
    assert modtrace.affine_parts(tm) is not None  # still recognised as A * score + B

    # mask: (q >= kv) & (q - kv <= 5), with lax's select_n / integer rem / trunc-div conventions exercised
    m = [Var() for _ in range(6)]
    mout = Var()
    mask_eqns = [eqn("ge", [q_, kv_], [m[0]]), eqn("sub", [q_, kv_], [m[1]]), eqn("le", [m[1], lit(5)], [m[2]]),
                 eqn("and", [m[0], m[2]], [m[3]]), eqn("rem", [m[1], lit(-3)], [m[4]]), eqn("eq", [m[4], lit(-7)], [m[5]]),
                 eqn("select_n", [m[5], m[3], lit(False)], [mout])]
    mj = NS(constvars=[], invars=[b_, h_, q_, kv_], outvars=[mout], eqns=mask_eqns)

    def run_mask():
        _, bb, hh, qq, kk = modtrace._leaf_syms()
        (res,) = jf._run_jaxpr(mj, [], [bb, hh, qq, kk])
        return modtrace.cast(modtrace._lift(res), modtrace.B1)

    tmask = modtrace._traced(None, run_mask, "mask")
    gm = np.broadcast_to(modtrace.evaluate(tmask, None, b, h, q, kv), s.shape)
    wm = np.broadcast_to(np.asarray(generate_sliding_window(5)(b, h, q, kv)).astype(bool), s.shape)
    assert np.array_equal(gm, wm)
    # C remainder takes the sign of the dividend (numpy's fmod), truncating division rounds to zero
    def run_rem():
        _, bb, hh, qq, kk = modtrace._leaf_syms()
        return modtrace.cast(modtrace._lift(jf._c_rem(qq - 9, 4) * 100 + jf._trunc_div(qq - 9, 4)), modtrace.F32)

    got = modtrace.evaluate(modtrace._traced(None, run_rem, "score"), s, b, h, q, kv)
    qv = (q - 9).astype(np.int64)
    want = np.fmod(qv, 4) * 100 + np.trunc(qv / 4).astype(np.int64)
    assert np.array_equal(np.broadcast_to(got, s.shape), np.broadcast_to(want, s.shape).astype(np.float32))


def test_jnp_mods_go_through_the_jaxpr_front_end():
    jax = pytest.importorskip("jax")
    import jax.numpy as jnp

    def alibi(score, b, h, q_idx, kv_idx):
        return score + (q_idx - kv_idx) * jnp.exp2(-((h + 1) * 8.0 / 8))

    tm = modtrace.lower_mods(alibi, None).score
    s, b, h, q, kv = _grid(H=8)
    got = modtrace.evaluate(tm, s, b, h, q, kv)
    want = np.asarray(generate_alibi_bias(8)(s, b, h, q, kv), dtype=np.float32)
    np.testing.assert_allclose(np.broadcast_to(got, want.shape), want, rtol=2e-6, atol=2e-6)


def test_bias_that_is_linear_in_an_index_gets_a_slope():
    """Relative-position biases (ALiBi) are linear in q and in kv: the lowering emits the slope so
    that the kernels add multiples of it along a tile instead of converting an integer per element.
    Mods that are not linear, or whose integer part could leave the range where the conversion to
    float is exact, get none."""
    from flaxattention_b200 import modtrace as mt
    from flaxattention_b200.mods import generate_alibi_bias

    ms = mt.lower_mods(generate_alibi_bias(8), None)
    assert "FA_SCORE_LINEAR_KV" in ms.source and "FA_SCORE_LINEAR_Q" in ms.source
    # slope along kv = -slope along q = -(2 ** -(h + 1)) * log2(e), whatever q and kv are
    import math
    for leaf, sign in (("kv", -1.0), ("q", 1.0)):
        root = ms.linear[leaf]
        for h in (0, 3, 7):
            got = float(mt.evaluate(mt.TracedMod("score", root, []), 0.0, 0, h, 5, 9))
            assert abs(got - sign * 2.0 ** -(h + 1) * math.log2(math.e)) < 1e-6

    def checkerboard(score, b, h, q_idx, kv_idx):
        return mt.where((q_idx - kv_idx) % 2 == 0, score * 0.5, score * 2.0)

    def quadratic(score, b, h, q_idx, kv_idx):
        d = mt.float32(q_idx - kv_idx)
        return score + d * d

    def huge(score, b, h, q_idx, kv_idx):
        return score + mt.float32(kv_idx * 1000000 + q_idx)

    for fn in (checkerboard, quadratic, huge):
        src = mt.lower_mods(fn, None).source
        assert "FA_SCORE_LINEAR_KV" not in src, fn.__name__
