"""The Tinapel design on the CPU: its configuration reader, the plain statement's own
mechanisms, and the engine's host logic (state slots, caches per pass, pages, batching)
with the kernels replaced by their plain statements (tests/host_ops.py)."""
import copy
import math

import pytest
import torch

import host_ops
import model_cases as mc
import plain_tinapel as plain
import tinapel_cases as tc
import traces
from inferx_b200.config.model_config import ConfigError
from inferx_b200.config.registry import config_from_json
from inferx_b200.engine.replay import ReplaySession

CASES = [("TA", tc.TA, 0, [5, 9, 17, 40, 3, 70], 4), ("TB", tc.TB, 1, [1, 6, 13, 31, 45, 80], 8),
         ("TC", tc.TC, 3, [21, 1, 50, 2, 37], 4)]
D = torch.float64


# -- configuration ---------------------------------------------------------------
def test_config_reads_every_size_and_constant():
    cfg, spec = config_from_json(tc.TA)
    assert (cfg.vocab, cfg.width, cfg.embedding_scale, cfg.norm_eps) == (200, 96, 3.0, 1e-6)
    assert (cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (0, 2, 3)
    g, a, w = (l.mixer for l in spec.layers)
    assert (g.heads, g.dim, g.vdim, g.tau, g.decay_rank) == (3, 8, 12, 4.0, 5)
    assert abs(g.q_scale - 8 ** -0.5) < 1e-15
    assert (a.heads, a.kv_heads, a.head_dim, a.scale, a.softcap, a.temp_coef, a.temp_every) == \
        (4, 2, 20, 0.3, 4.0, 0.5, 4)
    assert (w.heads, w.dim, w.decay_rank) == (2, 16, 6)
    f0, f2 = spec.layers[0].ffn, spec.layers[2].ffn
    assert spec.layers[1].ffn is None and spec.layers[1].post_norm is None
    assert (f0.num_experts, f0.top_k, f0.expert_intermediate, f0.routed_scale) == (4, 2, 24, 1.0)
    assert f0.shared.intermediate == 40 and f2.shared is None and f2.routed_scale == 2.5
    assert f0.renormalize and not f0.shared_gated
    # layers 0 and 1 three times, each pass with a cache of its own, then layer 2
    assert [(e.layer, e.cache_copy) for e in spec.schedule] == \
        [(0, 0), (1, 0), (0, 1), (1, 1), (0, 2), (1, 2), (2, 0)]
    befores = [e.before for e in spec.schedule]
    assert [b is not None for b in befores] == [True, False, True, False, True, False, False]
    assert [(b.row, b.embedding) for b in befores if b] == [(0, False), (1, True), (2, True)]
    assert spec.embed_scale == 3.0 and spec.tied_head and spec.final_norm.gain_offset == 1.0
    again, _ = config_from_json(cfg.to_json())
    assert again == cfg


def test_config_without_optional_parts():
    cfg, spec = config_from_json(tc.TB)
    assert not cfg.has_loop and all(e.before is None and e.cache_copy == 0 for e in spec.schedule)
    a = spec.layers[1].mixer
    assert a.softcap == 0.0 and a.temp_every == 0 and a.kv_heads == a.heads
    assert spec.layers[3].ffn is None


@pytest.mark.parametrize("change,match", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown kind"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=24), "values are the keys"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "do not split"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "of 4 experts"),
    (lambda c: c["loop"].update(stop=4), "does not fit"),
    (lambda c: c["layers"][0]["mixer"].update(heads="3"), "must be an integer"),
    (lambda c: c["layers"][0]["mixer"].pop("tau"), "'tau' is missing"),
    (lambda c: c.pop("width"), "'width' is missing"),
    (lambda c: c.update(layers=[]), "non-empty list"),
])
def test_config_refuses_what_it_cannot_run(change, match):
    cfg = copy.deepcopy(tc.TA)
    change(cfg)
    with pytest.raises(ConfigError, match=match):
        config_from_json(cfg)


def test_decay_rank_comes_from_the_checkpoint(tmp_path):
    """A configuration that does not state the inner size of the decays' low-rank
    products runs with whatever the folder's tensors have."""
    d = tc.make_model_dir(tc.TA, tmp_path / "m", 5)
    cfg, w = plain.read_model_folder(d)
    for layer in cfg["layers"]:
        layer["mixer"].pop("rank", None)
    import json
    with open(tmp_path / "m" / "config.json", "w") as f:
        json.dump(cfg, f)
    reqs = tc.make_requests(tc.TA, [11], 2)
    sess = ReplaySession(d, "float32", 64, page_size=4, max_live=1, device="cpu", ops=host_ops)
    rows = mc.run_trace(sess, traces.whole(reqs))
    mc.compare(rows, tc.reference_rows(d, reqs), 2e-5, "rank from the tensors")


# -- the plain statement's mechanisms ----------------------------------------------
def test_plain_norm_sinusoid_and_router():
    x = torch.tensor([[3.0, 4.0]], dtype=D)
    out = plain.norm_one_plus(x, torch.tensor([0.0, 1.0], dtype=D), 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(out, torch.tensor([[3 / r, 8 / r]], dtype=D))
    s = plain.sinusoid([0, 2], 4)
    assert torch.allclose(s[0], torch.tensor([0.0, 1.0, 0.0, 1.0], dtype=D))
    assert torch.allclose(s[1], torch.tensor([math.sin(2.0), math.cos(2.0), math.sin(0.02),
                                              math.cos(0.02)], dtype=D))
    w = {"m.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [-1.0, 0.0]], dtype=D)}
    mlp = {"router": {"experts": 3, "top": 2, "scale": 2.0}}
    idx, wt = plain.route(w, "m", mlp, torch.tensor([[math.log(3.0), 0.0]], dtype=D))
    # scores 3 : 1 : 1/3 before normalising; the best two, renormalised, times the scale
    assert idx.tolist() == [[0, 1]] and torch.allclose(wt, torch.tensor([[1.5, 0.5]], dtype=D))


def test_plain_recurrences_by_hand():
    """One head, one key channel, one value channel: the recurrences are scalar."""
    one = torch.ones(1, 1, dtype=D)
    h = torch.tensor([[1.0], [2.0]], dtype=D)
    w = {"p.q": one * 1.0, "p.k": one, "p.v": one, "p.g": one, "p.o": one, "p.norm": torch.ones(1, dtype=D),
         "p.a1": one, "p.a2": one * 0.0, "p.a2.b": torch.zeros(1, dtype=D)}
    m = {"heads": 1, "dim": 1, "vdim": 1, "tau": 1.0}
    # decay sigmoid(0) = 0.5: S1 = 1, S2 = 0.5 + 4 = 4.5; o = S q; rms norm makes it its sign
    out = plain.gla_mixer(w, "p", m, h, 0.0)
    assert torch.allclose(out[:, 0], torch.tensor([plain.silu(torch.tensor(1.0, dtype=D)),
                                                   plain.silu(torch.tensor(2.0, dtype=D))]))
    w = {"p.r": one, "p.k": one, "p.v": one, "p.g": one, "p.o": one, "p.norm": torch.ones(1, dtype=D),
         "p.w1": one * 0.0, "p.w2": one * 0.0, "p.w0": torch.zeros(1, dtype=D),
         "p.u": torch.tensor([[3.0]], dtype=D)}
    w.update({f"p.mu.{s}": torch.zeros(1, dtype=D) for s in "rkvgw"})
    # without the final norm: o1 = u k v r = 3, S1 = 1; o2 = (1 + 3*4) * 2 = 26
    S, outs = 0.0, []
    for x in (1.0, 2.0):
        outs.append((S + 3.0 * x * x) * x)
        S = math.exp(-1.0) * S + x * x
    assert outs == [3.0, 26.0]
    got = plain.wkv_mixer(w, "p", {"heads": 1, "dim": 1}, h, 0.0)
    assert torch.allclose(got[:, 0], torch.tensor([plain.silu(torch.tensor(1.0, dtype=D)),
                                                   plain.silu(torch.tensor(2.0, dtype=D))]))


def test_plain_shift_reads_the_previous_token():
    h = torch.tensor([[1.0, 1.0], [3.0, 5.0]], dtype=D)
    eye = torch.eye(2, dtype=D)
    w = {"p.r": eye, "p.k": eye, "p.v": eye, "p.g": eye, "p.o": eye, "p.norm": torch.ones(2, dtype=D),
         "p.w1": torch.zeros(1, 2, dtype=D), "p.w2": torch.zeros(2, 1, dtype=D),
         "p.w0": torch.zeros(2, dtype=D), "p.u": torch.ones(1, 2, dtype=D)}
    w.update({f"p.mu.{s}": torch.zeros(2, dtype=D) for s in "rkvw"})
    w["p.mu.g"] = torch.tensor([1.0, 0.5], dtype=D)
    # only the gate is shifted.  Token 0 sees zeros before it: its gate is [0, 0.5 * 1], so
    # channel 0 of its output is zero and channel 1 is not; token 1's gate reads
    # [1, (1 + 5) / 2]
    out = plain.wkv_mixer(w, "p", {"heads": 1, "dim": 2}, h, 0.0)
    assert out[0, 0] == 0 and out[0, 1] != 0
    assert out[1].abs().min() > 0


def test_plain_attention_temperature_steps_and_cap():
    """The temperature changes exactly where floor((p + 1) / every) does, and a capped
    score never exceeds the cap."""
    torch.manual_seed(0)
    T, Dh = 9, 4
    h = torch.randn(T, 6, dtype=D)
    w = {"p.q": torch.randn(Dh, 6, dtype=D), "p.k": torch.randn(Dh, 6, dtype=D),
         "p.q.norm": torch.ones(Dh, dtype=D), "p.k.norm": torch.ones(Dh, dtype=D),
         "p.o": torch.eye(Dh, dtype=D)}
    m = {"heads": 1, "kv_heads": 1, "dim": Dh, "scale": 1.0}
    base = plain.attention_mixer(w, "p", m, h, 1e-6)
    warm = plain.attention_mixer(w, "p", dict(m, q_temp={"coef": 0.7, "every": 4}), h, 1e-6)
    same = [bool(torch.allclose(base[p], warm[p])) for p in range(T)]
    assert same == [True, True, True, False, False, False, False, False, False]
    # a cap far below the scores' spread flattens the weights towards the mean of the values
    flat = plain.attention_mixer(w, "p", dict(m, softcap=1e-6), h, 1e-6)
    k_raw = h @ w["p.k"].T
    assert torch.allclose(flat[5], k_raw[:6].mean(0), atol=1e-5)


def test_each_pass_of_a_loop_keeps_a_state_of_its_own(tmp_path):
    d = tc.make_model_dir(tc.TC, tmp_path / "m", 1)
    sess = ReplaySession(d, "float32", 64, page_size=4, max_live=2, device="cpu", ops=host_ops)
    toks = tc.make_requests(tc.TC, [9], 0)["r0"]
    sess.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks, "want": []}], "end": []})
    model, storage = sess.runtime.model, sess.runtime.storage
    assert model.cache_units == [(0, 0), (1, 0), (2, 0), (1, 1)]
    first = storage.state[1]["recurrent_state"][sess.manager.slot("a")]
    second = storage.state[3]["recurrent_state"][sess.manager.slot("a")]
    assert first.abs().max() > 0 and second.abs().max() > 0 and not torch.equal(first, second)


# -- the engine's host logic ---------------------------------------------------------
@pytest.mark.parametrize("name,cfg,seed,lengths,page", CASES)
@pytest.mark.parametrize("kind", list(mc.TRACE_KINDS))
def test_replay_matches_plain(tmp_path, name, cfg, seed, lengths, page, kind):
    d = tc.make_model_dir(cfg, tmp_path / "m", seed)
    reqs = tc.make_requests(cfg, lengths, seed)
    ref = tc.reference_rows(d, reqs)
    steps = mc.TRACE_KINDS[kind](reqs)
    sess = ReplaySession(d, "float32", traces.peak_tokens(steps), page_size=page, max_live=4,
                         device="cpu", ops=host_ops)
    rows = mc.run_trace(sess, steps)
    mc.compare(rows, ref, 2e-5, f"{name}/{kind}")
    if kind in ("whole", "tail", "portions"):
        assert len(rows) == sum(lengths)


def test_state_slot_of_a_finished_request_starts_from_zero(tmp_path):
    """Two requests one after the other in a pool with one slot: the second must see
    neither the first one's recurrent state nor its last input."""
    d = tc.make_model_dir(tc.TA, tmp_path / "m", 2)
    reqs = tc.make_requests(tc.TA, [12, 9], 5)
    ref = tc.reference_rows(d, reqs)
    sess = ReplaySession(d, "float32", 64, page_size=4, max_live=1, device="cpu", ops=host_ops)
    rows = mc.run_trace(sess, traces.whole(reqs))
    mc.compare(rows, ref, 2e-5, "slot reuse")


def test_greedy_generation_through_the_engine(tmp_path):
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    d = tc.make_model_dir(tc.TB, tmp_path / "m", 4)
    c, w = plain.read_model_folder(d)
    prompts = list(tc.make_requests(tc.TB, [7, 19, 3], 8).values())
    eng = Engine.create(EngineConfig(model=d, dtype="float32", device="cpu", block_size=4,
                                     max_num_seqs=2, num_gpu_blocks_override=64,
                                     prefill_chunk=5, max_model_len=64), ops=host_ops)
    done = eng.generate([Request(p, SamplingParams(max_tokens=6, ignore_eos=True))
                         for p in prompts])
    for p, c_out in zip(prompts, done):
        seq = list(p)
        for _ in range(6):
            seq.append(int(plain.forward(w, c, seq)[-1].argmax()))
        assert c_out.output_tokens == seq[len(p):]


def test_preemption_rebuilds_state_and_cache(tmp_path):
    """A pool too small for all three requests: the preempted ones give back pages and
    slot, start again from position 0 in a zeroed slot, and generate the same tokens."""
    from inferx_b200 import Engine, EngineConfig, Request, SamplingParams
    d = tc.make_model_dir(tc.TA, tmp_path / "m", 0)
    reqs = tc.make_requests(tc.TA, [5, 9, 17], 0)

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
