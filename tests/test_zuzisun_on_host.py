"""The Zuzisun design on the CPU: its configuration reader, the plain statement's own
mechanisms, and the engine's host logic (state slots, pages, windows, batching) with the
kernels replaced by their plain statements (tests/host_ops.py)."""
import copy
import json
import math

import pytest
import torch

import host_ops
import model_cases as mc
import plain_zuzisun as plain
import traces
import zuzisun_cases as zc
from inferx_b200.config.model_config import ConfigError
from inferx_b200.config.registry import config_from_json
from inferx_b200.engine.replay import ReplaySession

CASES = [("ZA", zc.ZA, 0, [5, 9, 17, 40, 3, 70], 4), ("ZB", zc.ZB, 1, [1, 6, 13, 31, 45, 80], 8),
         ("ZD", zc.ZD, 3, [21, 1, 50, 2, 37], 4)]


# -- configuration ---------------------------------------------------------------
def test_config_reads_every_size_and_constant():
    cfg, spec = config_from_json(zc.ZA)
    assert (cfg.vocab, cfg.width, cfg.embedding_scale, cfg.norm_groups) == (200, 96, 2.0, 3)
    m0, m1 = spec.layers[0].mixer, spec.layers[1].mixer
    assert (m0.heads, m0.dim, m0.rot_dim, m0.vdim, m0.kv_rank, m0.window) == (3, 24, 16, 20, 40, 10)
    assert m0.position.scaling_factor == 8.0 and m0.position.original_context == 64
    assert m1.position.rotary_dim == 8 and m1.position.scaling_factor == 0.0 and m1.window == 7
    assert spec.layers[1].ffn is None and spec.layers[0].ffn.limit == 0.8
    assert spec.embed_scale == 2.0 and spec.tied_head and spec.final_norm.groups == 3
    assert [l.ffn.intermediate for l in spec.layers if l.ffn] == [112, 40]
    # what was read is what is written back
    again, _ = config_from_json(cfg.to_json())
    assert again == cfg


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="experts"), "unknown kind"),
    (lambda c: c["norm"].update(groups=5), "norm groups"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=18), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"].update(heads="3"), "must be an integer"),
    (lambda c: c.pop("width"), "'width' is missing"),
    (lambda c: c.update(layers=[]), "non-empty list"),
])
def test_config_refuses_what_it_cannot_run(change, match):
    cfg = copy.deepcopy(zc.ZA)
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        config_from_json(cfg)


# -- the plain statement's mechanisms ----------------------------------------------
def test_plain_grouped_norm_and_shift():
    v = torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=torch.float64)
    out = plain.grouped_rms_norm(v, torch.ones(4, dtype=torch.float64), 2, 0.0)
    r0, r1 = math.sqrt(12.5), math.sqrt(2.0)
    assert torch.allclose(out, torch.tensor([[3 / r0, 4 / r0, 0.0, 2 / r1]], dtype=torch.float64))
    h = torch.tensor([[1.0, 1.0], [3.0, 5.0]], dtype=torch.float64)
    mix = torch.tensor([0.5, 1.0], dtype=torch.float64)
    assert plain.token_shift(h, mix).tolist() == [[0.5, 0.0], [2.0, 1.0]]


def test_plain_rotation_and_window():
    f, mag = plain.rotary_frequencies(8, 100.0)
    assert mag == 1.0 and torch.allclose(f, torch.tensor([1.0, 100 ** -0.25, 0.1, 100 ** -0.75],
                                                         dtype=torch.float64))
    f2, mag2 = plain.rotary_frequencies(8, 100.0, {"factor": 4.0, "original": 16, "fast": 2.0,
                                                   "slow": 0.5})
    assert abs(mag2 - (0.1 * math.log(4.0) + 1.0)) < 1e-12
    # pairs below lo keep their frequency, above hi have it divided by the factor
    assert f2[0] == f[0] and abs(float(f2[-1]) - float(f[-1]) / 4.0) < 1e-12
    v = torch.tensor([[[1.0, 0.0, 7.0, 9.0]]], dtype=torch.float64)
    out = plain.rotate_interleaved(v, torch.tensor([1]), torch.tensor([math.pi / 2],
                                                                     dtype=torch.float64), 2.0)
    assert torch.allclose(out, torch.tensor([[[0.0, 2.0, 7.0, 9.0]]], dtype=torch.float64),
                          atol=1e-12)
    m = plain.window_mask(5, 3)
    assert m[4].tolist() == [False, False, True, True, True] and m[1].tolist()[:3] == [True, True, False]
    assert plain.window_mask(4, 0)[3].tolist() == [True] * 4


def test_plain_model_sees_exactly_its_window(tmp_path):
    """Changing a token just outside every layer's reach leaves the last logits alone;
    the reach of stacked windows and shifts is the sum over layers."""
    cfg = copy.deepcopy(zc.ZA)
    d = zc.make_model_dir(cfg, tmp_path / "m", 3)
    c, w = plain.read_model_folder(d)
    reach = sum(l["mixer"]["mask"]["size"] - 1 + 1 for l in c["layers"])   # window - 1, shift 1
    toks = zc.make_requests(cfg, [60], 1)["r0"]
    base = plain.forward(c, w, toks)[-1]
    far = list(toks)
    far[59 - reach - 1] = (far[59 - reach - 1] + 1) % cfg["vocab"]
    assert torch.equal(plain.forward(c, w, far)[-1], base)
    near = list(toks)
    near[59 - reach] = (near[59 - reach] + 1) % cfg["vocab"]
    assert not torch.equal(plain.forward(c, w, near)[-1], base)


# -- the engine's host logic ---------------------------------------------------------
@pytest.mark.parametrize("name,cfg,seed,lengths,page", CASES)
@pytest.mark.parametrize("kind", list(mc.TRACE_KINDS))
def test_replay_matches_plain(tmp_path, name, cfg, seed, lengths, page, kind):
    d = zc.make_model_dir(cfg, tmp_path / "m", seed)
    reqs = zc.make_requests(cfg, lengths, seed)
    ref = zc.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, "float32", traces.peak_tokens(steps), page_size=page, max_live=4,
                         device="cpu", ops=host_ops)
    rows = mc.run_trace(sess, steps)
    mc.compare(rows, ref, 2e-5, f"{name}/{kind}")
    if kind in ("whole", "tail", "portions"):
        assert len(rows) == sum(lengths)


def test_state_slot_of_a_finished_request_starts_from_zero(tmp_path):
    """Two requests one after the other in a pool with one slot: the second must not see
    the first one's last row as the token before its first."""
    d = zc.make_model_dir(zc.ZA, tmp_path / "m", 2)
    reqs = zc.make_requests(zc.ZA, [12, 9], 5)
    ref = zc.reference_rows(d, reqs)
    steps = traces.whole(reqs)
    sess = ReplaySession(d, "float32", 64, page_size=4, max_live=1, device="cpu", ops=host_ops)
    rows = mc.run_trace(sess, steps)
    mc.compare(rows, ref, 2e-5, "slot reuse")


def test_windowed_layers_give_pages_back(tmp_path):
    d = zc.make_model_dir(zc.ZA, tmp_path / "m", 2)
    toks = zc.make_requests(zc.ZA, [90], 6)["r0"]
    sess = ReplaySession(d, "float32", 128, page_size=4, max_live=1, device="cpu", ops=host_ops)
    sess.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": []})
    mgr = sess.manager
    assert [g.window for g in mgr.groups] == [7, 10]
    assert mgr.pages_held("a", 0) <= 3 and mgr.pages_held("a", 1) <= 4


def test_greedy_generation_through_the_engine(tmp_path):
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    d = zc.make_model_dir(zc.ZB, tmp_path / "m", 4)
    c, w = plain.read_model_folder(d)
    prompts = list(zc.make_requests(zc.ZB, [7, 19, 3], 8).values())
    eng = Engine.create(EngineConfig(model=d, dtype="float32", device="cpu", block_size=4,
                                     max_num_seqs=2, num_gpu_blocks_override=64,
                                     prefill_chunk=5, max_model_len=64), ops=host_ops)
    done = eng.generate([Request(p, SamplingParams(max_tokens=6, ignore_eos=True))
                         for p in prompts])
    for p, c_out in zip(prompts, done):
        seq = list(p)
        for _ in range(6):
            seq.append(int(plain.forward(c, w, seq)[-1].argmax()))
        assert c_out.output_tokens == seq[len(p):]


def test_preemption_rebuilds_shift_state_and_cache(tmp_path):
    """A pool too small for all three requests: the preempted ones give back pages and
    slot, start again from position 0 in a zeroed slot, and generate the same tokens."""
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    d = zc.make_model_dir(zc.ZB, tmp_path / "m", 0)
    reqs = zc.make_requests(zc.ZB, [5, 9, 17], 0)

    def run(pages):
        eng = Engine.create(EngineConfig(model=d, dtype="float32", device="cpu", block_size=4,
                                         max_num_seqs=3, num_gpu_blocks_override=pages,
                                         max_model_len=64), ops=host_ops)
        outs = eng.generate([Request(t, SamplingParams(max_tokens=8, ignore_eos=True))
                             for t in reqs.values()])
        return [c.output_tokens for c in outs], eng.stats()["preemptions"]
    roomy, p0 = run(64)
    tight, p1 = run(6)
    assert p0 == 0 and p1 >= 1 and roomy == tight
