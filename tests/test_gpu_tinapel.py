"""The Tinapel design on the GPU: every new kernel alone against its plain statement
(tests/host_ops.py), then the engine against the plain model (tests/plain_tinapel.py):
whole prompts, prefill against token-by-token decoding, portions down to two tokens,
unequal batches with pages and slots used again, long decoding with recorded steps, and
greedy generation through the engine's own entry point."""
import json
import os
import subprocess
import sys
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import host_ops
import model_cases as mc
import plain_tinapel as plain
import tinapel_cases as tc
import traces
from conftest import ROOT
from inferx_b200.engine.replay import ReplaySession

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def _ops():
    from inferx_b200.kernels import ops
    return ops


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2)


def _step(q_lens, starts, slots=None):
    """A batch description: sequence s brings q_lens[s] tokens from position starts[s]."""
    seq_of, pos, cu = [], [], [0]
    for s, (n, a) in enumerate(zip(q_lens, starts)):
        seq_of += [s] * n
        pos += list(range(a, a + n))
        cu.append(cu[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)
    return SimpleNamespace(
        seq_of_token=i32(seq_of), positions=i32(pos), cu_q=i32(cu), q_pos0=i32(list(starts)),
        q_lens=list(q_lens), num_seqs=len(q_lens), num_tokens=len(seq_of),
        kv_len=i32([a + n for n, a in zip(q_lens, starts)]),
        max_kv_len=max(a + n for n, a in zip(q_lens, starts)), max_q_len=max(q_lens),
        all_decode=all(n == 1 for n in q_lens), num_decode_seqs=0, cu_q_prompt=None,
        state_slot=i32(slots if slots is not None else list(range(len(q_lens)))))


def _cuda(ns):
    return SimpleNamespace(**{k: (v.cuda() if torch.is_tensor(v) else v)
                              for k, v in vars(ns).items()})


# -- kernels alone -------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [96, 1024, 51])
def test_embedding_with_sinusoid(dtype, width):
    g = torch.Generator().manual_seed(width)
    table = torch.randn(40, width, generator=g).to(dtype)
    ids = torch.tensor([3, 39, 0, 7, 7], dtype=torch.int32)
    pos = torch.tensor([0, 1, 4095, 17, 100000], dtype=torch.int32)
    i = torch.arange((width + 1) // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * i / width).float()
    ref = host_ops.embed_sinusoid(table, ids, pos, freq, 2.5)
    out = _ops().embed_sinusoid(table.cuda(), ids.cuda(), pos.cuda(), freq.cuda(), 2.5)
    torch.testing.assert_close(out.cpu(), ref, rtol=1e-5, atol=1e-5)
    # position 0 adds 0, 1, 0, 1, ...
    first = out[0].cpu() - table[3].float() * 2.5
    assert torch.allclose(first[0::2], torch.zeros_like(first[0::2]), atol=1e-5)
    assert torch.allclose(first[1::2], torch.ones_like(first[1::2]), atol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [96, 2048, 61, 7168])
def test_summed_norm_pair(dtype, width):
    g = torch.Generator().manual_seed(width)
    T = 7
    resid = torch.randn(T, width, generator=g)
    g1 = 1.0 + 0.3 * torch.randn(width, generator=g)
    g2 = 1.0 + 0.3 * torch.randn(width, generator=g)
    a = torch.randn(T, width, generator=g)                       # fp32 term
    b = torch.randn(T, width, generator=g).to(dtype)             # a term in the run's type
    c = torch.randn(T, width, generator=g)
    vec = torch.randn(width, generator=g)
    for terms, v, gains in (([a, b], None, (g1, g2)), ([a, b, c], vec, (g1,)), ([], vec, (g1, g2)),
                            ([], None, (g2,)), ([b], None, (g1, g2))):
        r_ref = resid.clone()
        ref = host_ops.add_rmsnorm_sum(r_ref, terms, v, gains, 1e-5, dtype)
        r = resid.cuda()
        out = _ops().add_rmsnorm_sum(r, [t.cuda() for t in terms],
                                     None if v is None else v.cuda(),
                                     tuple(x.cuda() for x in gains), 1e-5, dtype)
        assert len(out) == len(gains)
        torch.testing.assert_close(r.cpu(), r_ref, rtol=2e-6, atol=2e-6)
        for o, e in zip(out, ref):
            torch.testing.assert_close(o.cpu().float(), e.float(), **_tol(dtype))
    rows = torch.tensor([6, 0, 3, 3], dtype=torch.int32)
    ref = host_ops.add_rmsnorm_sum(resid.clone(), [a, b], vec, (g1,), 1e-5, dtype, rows=rows)
    r = resid.cuda()
    out = _ops().add_rmsnorm_sum(r, [a.cuda(), b.cuda()], vec.cuda(), (g1.cuda(),), 1e-5, dtype,
                                 rows=rows.cuda())
    torch.testing.assert_close(out[0].cpu().float(), ref[0].float(), **_tol(dtype))
    assert torch.equal(r.cpu(), resid)            # gathered rows leave the stream alone


@pytest.mark.parametrize("width", [96, 328, 50])
def test_summed_norm_takes_an_unwritten_mixture_output(width):
    """A mixture's output that was never written (expert rows, places, weights, shared
    part) is combined in the pass that adds and norms; the result is that of writing it
    out first."""
    ops = _ops()
    g = torch.Generator().manual_seed(width)
    T, k, dt = 9, 2, torch.bfloat16
    resid = torch.randn(T, width, generator=g)
    a = torch.randn(T, width, generator=g)
    y = torch.randn(T * k, width, generator=g).to(dt).cuda()
    dest = torch.randperm(T * k, generator=g).to(torch.int32).cuda()
    tw = torch.rand(T, k, generator=g).cuda()
    shared = torch.randn(T, width, generator=g).to(dt).cuda()
    g1 = (1.0 + 0.3 * torch.randn(width, generator=g)).cuda()
    g2 = (1.0 + 0.3 * torch.randn(width, generator=g)).cuda()
    for sh in (shared, None):
        pend = ops.CombinePending(y, dest, tw, sh, None)
        written = ops.moe_combine(y, dest, tw, sh, None)
        r1, r2 = resid.cuda(), resid.cuda()
        fused = ops.add_rmsnorm_sum(r1, [a.cuda(), pend], None, (g1, g2), 1e-5, dt)
        plain_ = ops.add_rmsnorm_sum(r2, [a.cuda(), written], None, (g1, g2), 1e-5, dt)
        # the written form rounds the combined row to bfloat16 first; the fused one does not
        torch.testing.assert_close(r1, r2, rtol=1e-2, atol=3e-2)
        ref = host_ops.add_rmsnorm_sum(resid.clone(), [a, host_ops.moe_combine(
            y.cpu(), dest.cpu(), tw.cpu(), None if sh is None else sh.cpu(), None).float()], None,
            (g1.cpu(), g2.cpu()), 1e-5, dt)
        for o, e, p_ in zip(fused, ref, plain_):
            torch.testing.assert_close(o.cpu().float(), e.float(), **_tol(dt))
            torch.testing.assert_close(o.float(), p_.float(), **_tol(dt))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,page", [(4, 2, 20, 4), (3, 1, 9, 8), (8, 8, 128, 16), (5, 5, 33, 2)])
def test_qk_norm_append(dtype, H, G, D, page):
    g = torch.Generator().manual_seed(D)
    step = _step([1, 6, 2], [130, 0, 5])
    T = 9
    qk = (torch.randn(T, (H + G) * D, generator=g) * 3.0).to(dtype)
    qg = 1.0 + 0.3 * torch.randn(D, generator=g)
    kg = 1.0 + 0.3 * torch.randn(D, generator=g)
    pages = 40
    slots = torch.randperm(pages * page, generator=g)[:T].to(torch.int32)
    kc = torch.zeros(pages, G, page, D, dtype=dtype)
    vc = torch.zeros_like(kc)
    for coef, every in ((0.0, 0), (0.4, 3), (0.25, 131)):
        kr, vr = kc.clone(), vc.clone()
        ref = host_ops.qk_norm_append(qk, qg, kg, step.positions, H, G, D, 1e-5, coef, every, kr,
                                      vr, slots)
        kd, vd = kc.cuda(), vc.cuda()
        out = _ops().qk_norm_append(qk.cuda(), qg.cuda(), kg.cuda(), step.positions.cuda(), H, G, D,
                                    1e-5, coef, every, kd, vd, slots.cuda())
        torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))
        torch.testing.assert_close(kd.cpu().float(), kr.float(), **_tol(dtype))
        assert torch.equal(vd.cpu(), vr)          # the values are the keys as projected
    # without caches nothing is written and the queries are the same
    out2 = _ops().qk_norm_append(qk.cuda(), qg.cuda(), kg.cuda(), step.positions.cuda(), H, G, D,
                                 1e-5, 0.25, 131, None, None, None)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [96, 1024, 50])
def test_shift_mix(dtype, width):
    g = torch.Generator().manual_seed(width)
    step = _step([1, 5, 2, 1], [7, 0, 3, 0], slots=[4, 0, 2, 5])
    T = 9
    x = torch.randn(T, width, generator=g).to(dtype)
    mu = torch.rand(5, width, generator=g) * 1.4 - 0.2
    state = torch.randn(6, width, generator=g)
    st_ref = state.clone()
    ref = host_ops.shift_mix(x, mu, st_ref, step)
    st = state.cuda()
    out = _ops().shift_mix(x.cuda(), mu.cuda(), st, _cuda(step))
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))
    torch.testing.assert_close(st.cpu(), st_ref, rtol=0, atol=0)     # the state is exact
    assert torch.equal(st_ref[1], state[1]) and torch.equal(st_ref[3], state[3])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,C,R", [(9, 136, 12), (1, 35, 3), (70, 512, 64), (17, 300, 1)])
def test_lowrank_decay(dtype, T, C, R):
    g = torch.Generator().manual_seed(C)
    wide = (torch.randn(T, R + 24, generator=g) * 2.0).to(dtype)
    x = wide[:, 24:]                      # a view into a wider projection
    w2 = torch.randn(R, C, generator=g)              # the outer matrix, transposed
    b = torch.randn(C, generator=g) * 2.0
    for mode, tau in (("exp_exp_tanh", 1.0), ("sigmoid_root", 12.0), ("sigmoid_root", 1.0)):
        ref = host_ops.lowrank_decay(x, w2, b, mode, tau)
        out = _ops().lowrank_decay(wide.cuda()[:, 24:], w2.cuda(), b.cuda(), mode, tau)
        torch.testing.assert_close(out.cpu(), ref, rtol=2e-5, atol=2e-6)
        assert float(out.min()) >= 0.0 and float(out.max()) <= 1.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,K,V", [(3, 8, 12), (2, 64, 64), (1, 40, 24), (5, 7, 7), (2, 128, 96),
                                   (4, 3, 5), (1, 200, 33)])
@pytest.mark.parametrize("bonus", [False, True])
def test_linear_recurrence(dtype, H, K, V, bonus):
    g = torch.Generator().manual_seed(K * V)
    step = _step([1, 37, 2, 1, 18], [7, 0, 3, 0, 100], slots=[4, 0, 2, 5, 1])
    T = 59
    wide = (torch.randn(T, 2 * H * K + H * V + 5, generator=g)).to(dtype)
    q, k, v = wide[:, :H * K], wide[:, H * K:2 * H * K], wide[:, 2 * H * K:2 * H * K + H * V]
    decay = torch.rand(T, H * K, generator=g) * 0.5 + 0.5
    u = torch.randn(H, K, generator=g) if bonus else None
    state = torch.randn(6, H, K, V, generator=g)
    st_ref = state.clone()
    ref = host_ops.linear_recurrence(q, k, v, decay, u, st_ref, step, H, K, V, 0.37, bonus)
    st = state.cuda()
    wd = wide.cuda()
    out = _ops().linear_recurrence(
        wd[:, :H * K], wd[:, H * K:2 * H * K], wd[:, 2 * H * K:2 * H * K + H * V], decay.cuda(),
        None if u is None else u.cuda(), st, _cuda(step), H, K, V, 0.37, bonus)
    scale = float(ref.abs().max())
    assert float((out.cpu() - ref).abs().max()) <= 2e-5 * scale
    assert float((st.cpu() - st_ref).abs().max()) <= 2e-5 * float(st_ref.abs().max())
    assert torch.equal(st.cpu()[3], state[3])     # a slot of no sequence is untouched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,K,V", [(2, 64, 64), (3, 20, 40), (1, 128, 33)])
@pytest.mark.parametrize("bonus", [False, True])
def test_linear_recurrence_in_segments(dtype, H, K, V, bonus):
    """Long portions are cut into segments that are walked side by side and joined: a long
    prompt beside a single token, a portion that continues a state, and one whose length is
    a segment and a token."""
    ops = _ops()
    g = torch.Generator().manual_seed(K + V)
    q_lens = [1, 700, 129, 65]
    step = _step(q_lens, [40, 0, 300, 0], slots=[3, 0, 2, 1])
    T = sum(q_lens)
    assert ops.recurrence_segments(step.max_q_len, len(q_lens), H, V)[1] > 1
    wide = (torch.randn(T, 2 * H * K + H * V, generator=g) * 0.5).to(dtype)
    q, k, v = wide[:, :H * K], wide[:, H * K:2 * H * K], wide[:, 2 * H * K:]
    decay = torch.rand(T, H * K, generator=g) * 0.2 + 0.8
    u = torch.randn(H, K, generator=g) if bonus else None
    state = torch.randn(4, H, K, V, generator=g)
    st_ref = state.clone()
    ref = host_ops.linear_recurrence(q, k, v, decay, u, st_ref, step, H, K, V, 0.5, bonus)
    st = state.cuda()
    wd = wide.cuda()
    out = ops.linear_recurrence(wd[:, :H * K], wd[:, H * K:2 * H * K], wd[:, 2 * H * K:],
                                decay.cuda(), None if u is None else u.cuda(), st, _cuda(step),
                                H, K, V, 0.5, bonus)
    assert float((out.cpu() - ref).abs().max()) <= 3e-5 * float(ref.abs().max())
    assert float((st.cpu() - st_ref).abs().max()) <= 3e-5 * float(st_ref.abs().max())


def test_linear_recurrence_does_not_depend_on_the_cut():
    """The same tokens in one step, in portions and one by one, alone and beside other
    sequences: the same bits, in the outputs and in the state."""
    ops = _ops()
    H, K, V, T = 3, 48, 40, 45
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(T, H * d, generator=g).to(torch.bfloat16).cuda() for d in (K, K, V))
    decay = (torch.rand(T, H * K, generator=g) * 0.3 + 0.7).cuda()
    u = torch.randn(H, K, generator=g).cuda()
    for bonus in (False, True):
        st0 = torch.zeros(3, H, K, V, device="cuda")
        whole = ops.linear_recurrence(q, k, v, decay, u, st0, _cuda(_step([T], [0], [1])), H, K, V,
                                      1.0, bonus)
        st1 = torch.zeros(3, H, K, V, device="cuda")
        parts, at = [], 0
        for n in (2, 17, 1, 16, 1, 1, 7):
            sl = slice(at, at + n)
            # beside another sequence that uses slot 0
            qq = torch.cat([q[:3], q[sl]]).contiguous()
            kk = torch.cat([k[:3], k[sl]]).contiguous()
            vv = torch.cat([v[:3], v[sl]]).contiguous()
            dd = torch.cat([decay[:3], decay[sl]]).contiguous()
            o = ops.linear_recurrence(qq, kk, vv, dd, u, st1,
                                      _cuda(_step([3, n], [0, at], [0, 1])), H, K, V, 1.0, bonus)
            parts.append(o[3:])
            at += n
        assert at == T
        assert torch.equal(torch.cat(parts), whole) and torch.equal(st1[1], st0[1])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,V,per_head", [(3, 12, False), (4, 64, True), (1, 33, True), (5, 7, False)])
def test_head_norm_gate(dtype, H, V, per_head):
    g = torch.Generator().manual_seed(V)
    T = 6
    o = torch.randn(T, H, V, generator=g) * 4.0
    gain = 1.0 + 0.3 * torch.randn(H * V if per_head else V, generator=g)
    wide = (torch.randn(T, H * V + 8, generator=g) * 2.0).to(dtype)
    ref = host_ops.head_norm_gate(o, gain, wide[:, 8:], 1e-5, dtype)
    out = _ops().head_norm_gate(o.cuda(), gain.cuda(), wide.cuda()[:, 8:], 1e-5, dtype)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))


@pytest.mark.parametrize("M", [1, 8, 13, 16, 17])
def test_batched_product_of_a_few_rows_against_large_matrices(M):
    """Up to 16 rows a matrix stream the weights; more go to the library; both are the
    batched product."""
    g = torch.Generator().manual_seed(M)
    x = (torch.randn(4, M, 1024, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(4, 1032, 1024, generator=g) * 0.05).to(torch.bfloat16)
    ref = torch.bmm(x.float(), w.float().transpose(1, 2))
    out = _ops().batched_linear(x.cuda(), w.cuda())
    assert out.shape == (4, M, 1032) and out.dtype == torch.bfloat16
    torch.testing.assert_close(out.cpu().float(), ref, rtol=1.6e-2, atol=1.6e-2)


def _kv_case(seed, H, G, D, page, q_lens, starts, dtype):
    g = torch.Generator().manual_seed(seed)
    step = _step(q_lens, starts)
    S = len(q_lens)
    need = [-(-(a + n) // page) for n, a in zip(q_lens, starts)]
    total = sum(need) + 3
    perm = torch.randperm(total, generator=g).to(torch.int32)
    bt = torch.full((S, max(need)), -1, dtype=torch.int32)
    at = 0
    for s, n in enumerate(need):
        bt[s, :n] = perm[at:at + n]
        at += n
    kc = (torch.randn(total, G, page, D, generator=g) * 0.3).to(dtype)
    vc = (torch.randn(total, G, page, D, generator=g)).to(dtype)
    q = (torch.randn(sum(q_lens), H, D, generator=g) * 0.3).to(dtype)
    return step, bt, kc, vc, q


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [20, 64, 128, 9])
@pytest.mark.parametrize("decode", [True, False])
def test_capped_attention_finds_one_key(dtype, D, decode):
    """One key carries a raw score far above the cap and a value of fives.  With the cap
    the output moves towards five by what exp(cap) is worth among hundreds of keys, for
    a key far back, on either side of a page border and at position 0; prompts and
    single tokens; every kernel form that takes the head size."""
    H, G, page, scale, cap = 4, 2, 16, 0.5, 6.0
    query_pos = 700
    for key_pos in (0, 16 * 40 - 1, 16 * 40, 333, 699, 700):
        q_lens, starts = ([1], [query_pos]) if decode else ([9], [query_pos - 8])
        step, bt, kc, vc, q = _kv_case(3, H, G, D, page, q_lens, starts, dtype)
        q[:] = q[-1, 0]
        qv = q[-1, 0].float()
        pg, off = bt[0, key_pos // page].long(), key_pos % page
        kc[pg, :, off] = (qv * (60.0 / scale) / (qv * qv).sum()).to(dtype)
        vc[pg, :, off] = 5.0
        ref = host_ops.paged_attention(q, kc, vc, bt, step, 0, scale, softcap=cap)
        out = _ops().paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), _cuda(step), 0,
                                     scale, softcap=cap).cpu().float()
        torch.testing.assert_close(out, ref.float(), **_tol(dtype))
        # exp(6) = 403 against about 700 keys with weights near 1: well between the two
        assert 1.0 < float(out[-1].mean()) < 4.0, (key_pos, float(out[-1].mean()))
        # uncapped, the same key takes everything
        free = _ops().paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), _cuda(step), 0,
                                      scale).cpu().float()
        assert float(free[-1].mean()) > 4.9


# -- the engine against the plain model ------------------------------------------------
CASES = [("TA", tc.TA, 0, [5, 9, 17, 40, 3, 70], 4), ("TB", tc.TB, 1, [1, 6, 13, 31, 45, 80], 8),
         ("TC", tc.TC, 3, [21, 1, 50, 2, 37], 4), ("TD", tc.TD, 2, [130, 2, 64, 33], 16)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg,seed,lengths,page", CASES)
@pytest.mark.parametrize("kind", list(mc.TRACE_KINDS))
def test_replay_matches_plain(tmp_path, dtype, name, cfg, seed, lengths, page, kind):
    d = tc.make_model_dir(cfg, tmp_path / "m", seed,
                          dtype="float32" if dtype == "float32" else "bfloat16")
    reqs = tc.make_requests(cfg, lengths, seed)
    ref = tc.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=page, max_live=4)
    rows = mc.run_trace(sess, steps)
    worst = mc.compare(rows, ref, tc.bound_for(dtype, d, reqs), f"{name}/{kind}/{dtype}")
    print(f"{name}/{kind}/{dtype}: worst relative error {worst:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_recorded_steps(tmp_path, dtype):
    """250 tokens one by one after a short prompt: the temperature passes many of its
    steps, the recurrent state and the previous input are carried through recorded steps,
    every pass of the loop in a state of its own."""
    cfg = tc.TA
    d = tc.make_model_dir(cfg, tmp_path / "m", 3,
                          dtype="float32" if dtype == "float32" else "bfloat16")
    reqs = tc.make_requests(cfg, [270], 3)
    ref = tc.reference_rows(d, reqs)
    steps = traces.tail_decode(reqs, 250)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=4, use_graphs=True)
    rows = mc.run_trace(sess, steps)
    assert len(rows) == 270 and sess.executor.graph_replays >= 200
    mc.compare(rows, ref, tc.bound_for(dtype, d, reqs), f"long decode {dtype}")


@pytest.mark.parametrize("dtype,kind", [("bfloat16", "whole"), ("bfloat16", "mixed"),
                                        ("float32", "tail")])
def test_long_prompts_at_tensor_core_sizes(tmp_path, dtype, kind):
    """Prompts of several hundred tokens at head sizes 64 and 128: the recurrence walks them
    in segments, attention runs on the tcgen05 and TMA kernels with squashed scores and cuts
    long contexts into runs, the temperature passes many of its steps."""
    cfg = tc.TD
    d = tc.make_model_dir(cfg, tmp_path / "m", 11,
                          dtype="float32" if dtype == "float32" else "bfloat16")
    reqs = tc.make_requests(cfg, [600, 260], 11)
    ref = tc.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=16, max_live=4)
    rows = mc.run_trace(sess, steps)
    sess.executor.poll_errors()
    mc.compare(rows, ref, tc.bound_for(dtype, d, reqs), f"long/{kind}/{dtype}")


def test_prefill_equals_decoding_in_32_bit(tmp_path):
    """The same sequence whole, token by token and in portions of two: the three runs
    agree with each other far inside their distance to the plain model."""
    cfg = tc.TC
    d = tc.make_model_dir(cfg, tmp_path / "m", 6)
    reqs = tc.make_requests(cfg, [75], 6)
    runs = []
    for steps in (traces.whole(reqs), traces.tail_decode(reqs, 74),
                  traces.portions(reqs, sizes=(2,))):
        sess = ReplaySession(d, "float32", 128, page_size=8, max_live=1)
        rows = mc.run_trace(sess, steps)
        runs.append(torch.stack([rows[("r0", p)] for p in range(75)]))
    scale = float(runs[0].abs().max())
    for other in runs[1:]:
        assert float((other - runs[0]).abs().max()) / scale < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(tmp_path, dtype):
    cfg = tc.TB
    d = tc.make_model_dir(cfg, tmp_path / "m", 5, dtype="bfloat16")
    reqs = tc.make_requests(cfg, [70, 33, 20, 9, 50, 41], 5)
    ref = tc.reference_rows(d, reqs)
    steps = traces.mixed(reqs, max_live=4, seed=1)
    out = tmp_path / "out"
    p = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
         "--out", str(out), "--max-tokens", str(traces.peak_tokens(steps))],
        input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True,
        timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    outs = []
    for s in steps:
        n = sum(len(e["want"]) for e in s["entries"])
        outs.append(None if n == 0 else torch.from_numpy(
            np.fromfile(out / f"{s['step']}.f32", dtype="<f4").reshape(n, cfg["vocab"]).copy()))
    rows = traces.collect(steps, outs)
    mc.compare(rows, ref, tc.bound_for(dtype, d, reqs), f"trace_run/{dtype}")


def test_greedy_generation_through_the_engine(tmp_path):
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    d = tc.make_model_dir(tc.TA, tmp_path / "m", 4)
    c, w = plain.read_model_folder(d)
    prompts = list(tc.make_requests(tc.TA, [7, 19, 3, 30, 11], 8).values())
    eng = Engine.create(EngineConfig(model=d, dtype="float32", block_size=4, max_num_seqs=3,
                                     num_gpu_blocks_override=96, prefill_chunk=6,
                                     max_model_len=64))
    done = eng.generate([Request(p, SamplingParams(max_tokens=12, ignore_eos=True))
                         for p in prompts])
    for p, c_out in zip(prompts, done):
        seq = list(p)
        for tok in c_out.output_tokens:
            lg = plain.forward(w, c, seq)[-1]
            top = torch.topk(lg, 2).values
            # the engine's choice is the plain model's, unless the two best are a tie in fp32
            assert tok == int(lg.argmax()) or float(top[0] - top[1]) < 1e-4 * float(lg.abs().max())
            seq.append(tok)
        assert len(c_out.output_tokens) == 12
