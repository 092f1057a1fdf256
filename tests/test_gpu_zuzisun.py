"""The Zuzisun design on the GPU: every new kernel alone against its plain statement
(tests/host_ops.py), then the engine against the plain model (tests/plain_zuzisun.py):
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
import plain_zuzisun as plain
import traces
import zuzisun_cases as zc
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
    return SimpleNamespace(seq_of_token=i32(seq_of), positions=i32(pos), cu_q=i32(cu),
                           q_pos0=i32(list(starts)), q_lens=list(q_lens),
                           state_slot=i32(slots if slots is not None else list(range(len(q_lens)))))


def _cuda(ns):
    return SimpleNamespace(**{k: (v.cuda() if torch.is_tensor(v) else v)
                              for k, v in vars(ns).items()})


# -- kernels alone -------------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [96, 1024, 50])
def test_token_shift(dtype, width):
    g = torch.Generator().manual_seed(width)
    step = _step([1, 5, 2, 1], [7, 0, 3, 0], slots=[4, 0, 2, 5])
    T = 9
    resid = torch.randn(T, width, generator=g)
    mix = torch.rand(width, generator=g) * 1.4 - 0.2
    state = torch.randn(6, width, generator=g)
    st_ref = state.clone()
    ref = host_ops.token_shift(resid, mix, st_ref, step, dtype)
    st = state.cuda()
    out = _ops().token_shift(resid.cuda(), mix.cuda(), st, _cuda(step), dtype)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))
    torch.testing.assert_close(st.cpu(), st_ref, rtol=0, atol=0)     # the state is exact
    assert torch.equal(st_ref[1], state[1]) and torch.equal(st_ref[3], state[3])   # others untouched


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width,groups", [(96, 3), (128, 1), (2048, 8), (60, 60), (7168, 2)])
def test_grouped_norm(dtype, width, groups):
    g = torch.Generator().manual_seed(groups)
    T = 11
    resid = torch.randn(T, width, generator=g)
    gain = 1.0 + 0.3 * torch.randn(width, generator=g)
    for delta_dtype in (torch.float32, dtype):
        delta = (torch.randn(T, width, generator=g) * 3.0).to(delta_dtype)
        r_ref = resid.clone()
        c_ref = host_ops.group_norm_add(r_ref, delta, gain, groups, 1e-5, dtype)
        r = resid.cuda()
        c = _ops().group_norm_add(r, delta.cuda(), gain.cuda(), groups, 1e-5, dtype)
        torch.testing.assert_close(r.cpu(), r_ref, rtol=2e-5, atol=2e-5)
        torch.testing.assert_close(c.cpu().float(), c_ref.float(), **_tol(dtype))
        assert _ops().group_norm_add(r, delta.cuda(), gain.cuda(), groups, 1e-5) is None
    rows = torch.tensor([10, 0, 3, 3], dtype=torch.int32)
    ref = host_ops.group_norm_rows(resid, rows, gain, groups, 1e-5, dtype)
    out = _ops().group_norm_rows(resid.cuda(), rows.cuda(), gain.cuda(), groups, 1e-5, dtype)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))
    out = _ops().group_norm_rows(resid.cuda(), None, gain.cuda(), groups, 1e-5, dtype)
    torch.testing.assert_close(out.cpu().float(),
                               host_ops.group_norm_rows(resid, None, gain, groups, 1e-5,
                                                        dtype).float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(5, 112), (3, 37), (16, 1024), (40, 1024)])
def test_clamped_glu(dtype, T, I):
    g = torch.Generator().manual_seed(I)
    gu = (torch.randn(T, 2 * I, generator=g) * 2.0).to(dtype)      # far beyond the limit too
    ref = host_ops.glu_clamped(gu, 0.9, 1.702, 1.0)
    out = _ops().glu_clamped(gu.cuda(), 0.9, 1.702, 1.0)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))
    assert float(ref.float().max()) <= 0.9 * 1.9 + 0.02                # both clamps acted
    if dtype == torch.bfloat16 and I % 8 == 0:
        w = (torch.randn(2 * I, 64, generator=g) * 0.4).to(dtype)
        x = torch.randn(T, 64, generator=g).to(dtype)
        ref = host_ops.glu_clamped(host_ops.linear(x, w), 0.9, 1.702, 1.0)
        out = _ops().gate_up_glu_clamped(x.cuda(), w.cuda(), 0.9, 1.702, 1.0)
        torch.testing.assert_close(out.cpu().float(), ref.float(), rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_output_gate(dtype):
    g = torch.Generator().manual_seed(1)
    H, T, D, off = 3, 7, 20, 33
    o = torch.randn(H, T, D, generator=g).to(dtype)
    proj = (torch.randn(T, off + H * D + 5, generator=g) * 3).to(dtype)
    ref = host_ops.gate_heads(o, proj, off)
    out = _ops().gate_heads(o.cuda(), proj.cuda(), off)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,dn,dr,rot_dims,rank", [(3, 24, 16, 16, 40), (2, 8, 24, 8, 24),
                                                  (16, 48, 32, 32, 256), (1, 5, 6, 2, 7)])
def test_latent_prepare(dtype, H, dn, dr, rot_dims, rank):
    g = torch.Generator().manual_seed(rank)
    step = _step([4, 1, 3], [0, 900, 61])
    T, page, P = 8, 4, 300
    q_off, kv_off = 3, 3 + H * (dn + dr) + 2
    proj = torch.randn(T, kv_off + rank + dr + 4, generator=g).to(dtype)
    freq = torch.rand(rot_dims // 2, generator=g)
    gain = 1.0 + 0.2 * torch.randn(rank, generator=g)
    slots = torch.randperm(P * page, generator=g)[:T].to(torch.int32)
    cache = torch.zeros(P, 1, page, rank + dr, dtype=dtype)
    c_ref = cache.clone()
    ref, ref_plain = host_ops.latent_prepare(proj, q_off, kv_off, step.positions, freq, 1.3, gain,
                                             1e-5, H, dn, dr, rot_dims, rank, c_ref, slots)
    c = cache.cuda()
    out, plain_part = _ops().latent_prepare(proj.cuda(), q_off, kv_off, step.positions.cuda(), freq.cuda(),
                                1.3, gain.cuda(), 1e-5, H, dn, dr, rot_dims, rank, c, slots.cuda())
    # angles reach 900 radians: fp32 cos/sin of an fp32 product on both sides
    tol = dict(rtol=2e-4, atol=2e-4) if dtype == torch.float32 else _tol(dtype)
    torch.testing.assert_close(out.cpu().float(), ref.float(), **tol)
    assert torch.equal(plain_part.cpu(), ref_plain)
    torch.testing.assert_close(c.cpu().float(), c_ref.float(), **tol)
    # without a cache only the queries are produced
    out2, _ = _ops().latent_prepare(proj.cuda(), q_off, kv_off, step.positions.cuda(),
                                    freq.cuda(), 1.3, gain.cuda(), 1e-5, H, dn, dr, rot_dims, rank,
                                    None, None)
    assert torch.equal(out2, out)


@pytest.mark.parametrize("M", [1, 8, 16, 40])
def test_products_batched_over_heads(M):
    """A few rows per head go through the weight-streaming kernel, more through the
    library; both against the plain product."""
    g = torch.Generator().manual_seed(M)
    for dtype, B, N, K in ((torch.bfloat16, 16, 512, 128), (torch.bfloat16, 5, 40, 24),
                           (torch.float32, 3, 20, 40)):
        x = torch.randn(B, M, K, generator=g).to(dtype)
        w = (torch.randn(B, N, K, generator=g) * 0.2).to(dtype)
        ref = host_ops.batched_linear(x, w)
        out = _ops().batched_linear(x.cuda(), w.cuda())
        torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))


@pytest.mark.parametrize("M", [1, 7, 16])
def test_clamped_glu_fused_into_the_small_product(M):
    g = torch.Generator().manual_seed(M)
    I, K = 320, 256
    w = (torch.randn(2 * I, K, generator=g) * 0.2).to(torch.bfloat16)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    ref = host_ops.glu_clamped(host_ops.linear(x.float(), w.float()), 1.1, 1.702, 1.0)
    out = _ops().gate_up_glu_clamped(x.cuda(), w.cuda(), 1.1, 1.702, 1.0)
    torch.testing.assert_close(out.cpu().float(), ref, rtol=2e-2, atol=2e-2)
    assert float(out.float().max()) > 1.0


def _attention_case(seed, H, rank, dr, page, q_lens, starts, dtype, spread=1.0):
    g = torch.Generator().manual_seed(seed)
    step = _step(q_lens, starts)
    T = sum(q_lens)
    kv = [a + n for a, n in zip(starts, q_lens)]
    maxb = max(-(-n // page) for n in kv)
    P = sum(-(-n // page) for n in kv) + 3
    perm = torch.randperm(P, generator=g)
    bt = torch.full((len(kv), maxb), -1, dtype=torch.int32)
    nxt = 0
    for s, n in enumerate(kv):
        for b in range(-(-n // page)):
            bt[s, b] = perm[nxt]
            nxt += 1
    cache = (torch.randn(P, 1, page, rank + dr, generator=g) * spread).to(dtype)
    q_lat = (torch.randn(H, T, rank, generator=g) * spread).to(dtype)
    q_rot = (torch.randn(T, H, dr, generator=g) * spread).to(dtype)
    return step, bt, cache, q_lat, q_rot


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,rank,dr,page,window", [(3, 40, 16, 4, 10), (5, 48, 8, 8, 0),
                                                   (16, 256, 32, 16, 100), (8, 128, 48, 16, 90),
                                                   (1, 7, 6, 16, 3), (9, 160, 0, 32, 50),
                                                   (70, 64, 16, 8, 33), (5, 512, 64, 16, 0),
                                                   (64, 128, 0, 16, 77)])
def test_latent_attention_unequal_batch(dtype, H, rank, dr, page, window):
    """Single tokens far into their sequences beside portions that start anywhere; every
    kernel form that takes the sizes."""
    step, bt, cache, q_lat, q_rot = _attention_case(
        rank, H, rank, dr, page, [1, 1, 37, 2, 64, 5], [333, 0, 0, 129, 70, 15], dtype, 0.5)
    ref = host_ops.latent_attention(q_lat, q_rot, cache, bt, step, window, 0.2)
    forms = ["general"]
    if dtype == torch.bfloat16 and rank in (64, 128, 256, 512) and dr % 16 == 0:
        forms.append("mma")
        assert _ops()._mma_latent_applies(q_lat.cuda(), q_rot.cuda())
    for form in forms:
        out = _ops().latent_attention(q_lat.cuda(), q_rot.cuda(), cache.cuda(), bt.cuda(),
                                      _cuda(step), window, 0.2, kernel=form)
        torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("page", [4, 16])
@pytest.mark.parametrize("decode", [True, False])
def test_latent_attention_finds_one_key(dtype, page, decode):
    """One key carries a score far above the rest and a latent of fives; the output is
    fives exactly when that key is visible: far back among hundreds, on either side of a
    page border, the oldest key of the window and the one just outside it, position 0."""
    H, rank, dr, window, scale = 2, 64, 16, 150, 0.5
    query_pos = 700
    forms = ["general", "mma"] if dtype == torch.bfloat16 else ["general"]
    for key_pos, seen in [(700 - 149, True), (700 - 150, False), (0, False), (700, True),
                          (699, True), (16 * 40 - 1, True), (16 * 40, True)]:
        q_lens, starts = ([1], [query_pos]) if decode else ([9], [query_pos - 8])
        step, bt, cache, q_lat, q_rot = _attention_case(3, H, rank, dr, page, q_lens, starts,
                                                        dtype, 0.1)
        q_rot[:] = q_rot[-1, 0]
        rec = cache[bt[0, key_pos // page].long(), 0, key_pos % page]
        qv = q_rot[-1, 0].float()
        rec[rank:] = (qv * (40.0 / scale) / (qv * qv).sum()).to(dtype)
        rec[:rank] = 5.0
        ref = host_ops.latent_attention(q_lat, q_rot, cache, bt, step, window, scale)
        for form in forms:
            out = _ops().latent_attention(q_lat.cuda(), q_rot.cuda(), cache.cuda(), bt.cuda(),
                                          _cuda(step), window, scale, kernel=form).cpu().float()
            torch.testing.assert_close(out, ref.float(), **_tol(dtype))
            last = out[:, -1]
            assert (last.mean() > 4.5) == seen, (form, key_pos, float(last.mean()))
    # no window: position 0 is seen from anywhere
    step, bt, cache, q_lat, q_rot = _attention_case(3, H, rank, dr, page, [1], [query_pos], dtype,
                                                    0.1)
    q_rot[:] = q_rot[-1, 0]
    rec = cache[bt[0, 0].long(), 0, 0]
    qv = q_rot[-1, 0].float()
    rec[rank:] = (qv * (40.0 / scale) / (qv * qv).sum()).to(dtype)
    rec[:rank] = 5.0
    out = _ops().latent_attention(q_lat.cuda(), q_rot.cuda(), cache.cuda(), bt.cuda(), _cuda(step),
                                  0, scale).cpu().float()
    assert out.mean() > 4.5


@pytest.mark.parametrize("window", [0, 1500])
@pytest.mark.parametrize("H,rank,dr", [(16, 512, 64), (8, 128, 32), (70, 64, 16)])
def test_latent_attention_single_tokens_over_long_contexts(window, H, rank, dr):
    """A few single tokens late in long sequences: the tensor-core form cuts the keys into
    chunks and merges the partial results."""
    dtype = torch.bfloat16
    step, bt, cache, q_lat, q_rot = _attention_case(5, H, rank, dr, 16, [1, 1, 1],
                                                    [2999, 37, 1700], dtype, 0.3)
    step.max_kv_len = 3000
    ref = host_ops.latent_attention(q_lat, q_rot, cache, bt, step, window, 0.1)
    for form in ("general", "mma"):
        out = _ops().latent_attention(q_lat.cuda(), q_rot.cuda(), cache.cuda(), bt.cuda(),
                                      _cuda(step), window, 0.1, kernel=form)
        torch.testing.assert_close(out.cpu().float(), ref.float(), **_tol(dtype))


def test_latent_attention_row_does_not_depend_on_its_batch():
    """The same query over the same keys gives the same bits alone, after other
    sequences, and as the last token of a portion."""
    ops = _ops()
    for (H, rank, dr, page), form in (((4, 40, 16, 8), "general"), ((4, 128, 16, 8), "general"),
                                      ((4, 128, 16, 8), "mma"), ((20, 256, 32, 16), "mma")):
        step, bt, cache, q_lat, q_rot = _attention_case(9, H, rank, dr, page, [1, 6, 1],
                                                        [50, 200, 90], torch.bfloat16, 0.5)
        full = ops.latent_attention(q_lat.cuda(), q_rot.cuda(), cache.cuda(), bt.cuda(),
                                    _cuda(step), 20, 0.3, kernel=form)
        alone = _step([1], [205])
        one = ops.latent_attention(q_lat[:, 6:7].contiguous().cuda(),
                                   q_rot[6:7].contiguous().cuda(), cache.cuda(),
                                   bt[1:2].contiguous().cuda(), _cuda(alone), 20, 0.3, kernel=form)
        assert torch.equal(full[:, 6], one[:, 0]), (H, rank, form)


# -- the engine against the plain model ------------------------------------------------
CASES = [("ZA", zc.ZA, 0, [5, 9, 17, 40, 3, 70], 4), ("ZB", zc.ZB, 1, [1, 6, 13, 31, 45, 80], 8),
         ("ZC", zc.ZC, 2, [130, 2, 64, 33], 16), ("ZD", zc.ZD, 3, [21, 1, 50, 2, 37], 4),
         ("ZE", zc.ZE, 4, [150, 3, 77, 40], 16)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,cfg,seed,lengths,page", CASES)
@pytest.mark.parametrize("kind", list(mc.TRACE_KINDS))
def test_replay_matches_plain(tmp_path, dtype, name, cfg, seed, lengths, page, kind):
    d = zc.make_model_dir(cfg, tmp_path / "m", seed,
                          dtype="float32" if dtype == "float32" else "bfloat16")
    reqs = zc.make_requests(cfg, lengths, seed)
    ref = zc.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=page, max_live=4)
    rows = mc.run_trace(sess, steps)
    worst = mc.compare(rows, ref, zc.bound_for(dtype, d, reqs), f"{name}/{kind}/{dtype}")
    print(f"{name}/{kind}/{dtype}: worst relative error {worst:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_recorded_steps(tmp_path, dtype):
    """250 tokens one by one after a short prompt: windows slide over many pages, pages
    are given back, the shift state is carried through recorded steps."""
    cfg = zc.ZA
    d = zc.make_model_dir(cfg, tmp_path / "m", 3,
                          dtype="float32" if dtype == "float32" else "bfloat16")
    reqs = zc.make_requests(cfg, [270], 3)
    ref = zc.reference_rows(d, reqs)
    steps = traces.tail_decode(reqs, 250)
    sess = ReplaySession(d, dtype, traces.peak_tokens(steps), page_size=4, use_graphs=True)
    rows = mc.run_trace(sess, steps)
    assert len(rows) == 270 and sess.executor.graph_replays >= 200
    mc.compare(rows, ref, zc.bound_for(dtype, d, reqs), f"long decode {dtype}")


def test_prefill_equals_decoding_in_32_bit(tmp_path):
    """The same sequence whole, token by token and in portions of two: the three runs
    agree with each other far inside their distance to the plain model."""
    cfg = zc.ZB
    d = zc.make_model_dir(cfg, tmp_path / "m", 6)
    reqs = zc.make_requests(cfg, [75], 6)
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
    cfg = zc.ZB
    d = zc.make_model_dir(cfg, tmp_path / "m", 5, dtype="bfloat16")
    reqs = zc.make_requests(cfg, [70, 33, 20, 9, 50, 41], 5)
    ref = zc.reference_rows(d, reqs)
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
    mc.compare(rows, ref, zc.bound_for(dtype, d, reqs), f"trace_run/{dtype}")


def test_greedy_generation_through_the_engine(tmp_path):
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    d = zc.make_model_dir(zc.ZA, tmp_path / "m", 4)
    c, w = plain.read_model_folder(d)
    prompts = list(zc.make_requests(zc.ZA, [7, 19, 3, 30, 11], 8).values())
    eng = Engine.create(EngineConfig(model=d, dtype="float32", block_size=4, max_num_seqs=3,
                                     num_gpu_blocks_override=96, prefill_chunk=6,
                                     max_model_len=64))
    done = eng.generate([Request(p, SamplingParams(max_tokens=12, ignore_eos=True))
                         for p in prompts])
    for p, c_out in zip(prompts, done):
        seq = list(p)
        for tok in c_out.output_tokens:
            lg = plain.forward(c, w, seq)[-1]
            top = torch.topk(lg, 2).values
            # the engine's choice is the plain model's, unless the two best are a tie in fp32
            assert tok == int(lg.argmax()) or float(top[0] - top[1]) < 1e-4 * float(lg.abs().max())
            seq.append(tok)
        assert len(c_out.output_tokens) == 12
