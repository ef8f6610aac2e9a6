"""Risepel layer-list decoders through the engine (driven sequences and the scheduler) against the float64 oracle.

Every test builds its own small configuration and random bf16-representable weights (oracle/risepel_ref.py); the engine
runs them in its exact mode (fp32 weights, cache and products) where a one-token slip of a window, a lost state or a
missing sink must show, and in its serving mode (bf16 weights / cache rows / GEMM operands) with a rounding-sized bound.
"""
import numpy as np
import pytest

import helix_b200 as hb
from helix_b200 import weights_io
from helix_b200.engine import CAPTURE_PROMPT_LOGITS, CAPTURE_STEP_LOGITS
from oracle import risepel_ref as ref
from oracle.weights import to_bf16_f32

pytestmark = pytest.mark.gpu

TOL = {1: 2e-4, 0: 6e-2}  # compute_f32 -> bound on rms(diff) / rms(expected) per logits row


def row_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    return np.sqrt((d * d).mean(-1)) / np.sqrt((want * want).mean(-1))


def make_engine(cfg, sd, f32, max_seqs=4, ctx=512, pool=0, batched=0, **kw):
    desc = weights_io.risepel_desc(cfg, {k: v.shape for k, v in sd.items()}, compute_f32=bool(f32))
    e = hb.Engine(hb.EngineConfig(device=0, max_seqs=max_seqs, max_ctx=ctx, max_batched_tokens=batched or ctx,
                                  kv_pool_tokens=pool, **kw))
    e.load_state_dict(desc, sd)
    return e


def tokens(seed, n, vocab):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()


def replay(e, toks, cuts):
    """Feed one sequence in portions of the given sizes (the rest one token at a time), all positions wanted."""
    sid, out, at = e.seq_open(), [], 0
    cuts = list(cuts)
    while at < len(toks):
        n = min(cuts.pop(0) if cuts else 1, len(toks) - at)
        out.append(e.seq_step([(sid, toks[at:at + n], list(range(n)))]))
        at += n
    e.seq_close(sid)
    return np.concatenate(out)


CONFIGS = {
    "gla_only": dict(order=("gla", "gla"), mlp_on=()),
    "latent_only": dict(order=("latent_attention",), mlp_on=()),
    "latent_ff": dict(order=("latent_attention", "latent_attention"), share=False),
    "mixed_shared": dict(),
    "one_head_alpha1": dict(alpha=1.0, gla=dict(heads=1, dim=32, vdim=8), lat=dict(heads=1, dim=8, vdim=16, window=7), cap=0.0),
    "ff_everywhere": dict(order=("gla", "latent_attention", "gla"), mlp_on=("gla", "latent_attention"), gla=dict(heads=2, dim=40, vdim=72)),
    # nothing a multiple of 8 or 4: every product takes the CUDA-core GEMM, rows are loaded element by element
    "odd_sizes": dict(width=90, gla=dict(heads=2, dim=12, vdim=20), lat=dict(heads=2, dim=12, vdim=20, kv_rank=28, q_rank=20, rot_dim=6, window=9), ff=50),
    # a vocabulary that is no multiple of 4, 200 key channels per GLA head (the widest state block), one value column
    "wide_state": dict(vocab=131, gla=dict(heads=1, dim=200, vdim=33), order=("gla", "latent_attention"), lat=dict(window=3)),
    "wide_rows": dict(width=128, vocab=256, lat=dict(heads=5, dim=16, vdim=8, kv_rank=72, q_rank=24, rot_dim=8, window=65), ff=64),
}


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_oracle(name, f32):
    cfg = ref.random_config(**CONFIGS[name])
    sd = ref.random_state_dict(cfg, seed=3)
    toks = tokens(1, 150, cfg["vocab"])  # crosses two page borders and every window of the configurations above
    want = ref.RisepelOracle(cfg, sd).forward(toks)
    with make_engine(cfg, sd, f32) as e:
        got = replay(e, toks, [len(toks)])
    assert row_err(got, want).max() < TOL[f32]


def test_partial_rotation_and_two_cache_planes():
    # rope on fewer entries than the rotated part holds; two attention layers with cache rows of different length
    cfg = ref.random_config(order=("latent_attention", "gla", "latent_attention"), share=False)
    cfg["layers"][0]["mixer"]["rot"]["dims"] = 8
    m = cfg["layers"][2]["mixer"]
    m.update(kv_rank=40, rot_dim=24, rot=dict(base=500.0, dims=24), dim=16, scale=0.2, mask=dict(size=33))
    sd = ref.random_state_dict(cfg, seed=5)
    toks = tokens(2, 100, cfg["vocab"])
    want = ref.RisepelOracle(cfg, sd).forward(toks)
    with make_engine(cfg, sd, 1) as e:
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[1]
        assert row_err(replay(e, toks, [37, 2, 31]), want).max() < TOL[1]


@pytest.mark.parametrize("f32", [1, 0])
def test_prefill_portions_and_single_tokens_agree(f32):
    cfg = ref.random_config()
    sd = ref.random_state_dict(cfg, seed=7)
    toks = tokens(3, 140, cfg["vocab"])
    want = ref.RisepelOracle(cfg, sd).forward(toks)
    with make_engine(cfg, sd, f32) as e:
        whole = replay(e, toks, [len(toks)])
        for cuts in ([64, 64], [63, 2, 2, 61], [19, 20, 21, 2, 45], [1, 1, 1, 2, 3, 64, 5], []):
            got = replay(e, toks, cuts)
            assert row_err(got, want).max() < TOL[f32], cuts
            # the same positions, cut differently: rounding only
            assert row_err(got, whole).max() < (1e-5 if f32 else 3e-2), cuts


def sharpen(sd, factor=6.0):
    """Peaked softmax: single keys dominate, so a key wrongly seen or missed moves the logits by far more than rounding."""
    return {k: to_bf16_f32(np.asarray(v) * (factor if k.endswith("mix.uq") else 1.0)) for k, v in sd.items()}


@pytest.mark.parametrize("window", [5, 64, 65, 70])
def test_window_edges_in_prompts_and_decoding(window):
    cfg = ref.random_config(order=("latent_attention",), mlp_on=(), lat=dict(window=window))
    sd = sharpen(ref.random_state_dict(cfg, seed=11))
    toks = tokens(4, 2 * 64 + 20, cfg["vocab"])
    want = ref.RisepelOracle(cfg, sd).forward(toks)
    # the oracle with a window one token longer / shorter is far away at the positions where the window has filled
    for dw in (-1, 1):
        c2 = ref.random_config(order=("latent_attention",), mlp_on=(), lat=dict(window=window + dw))
        other = ref.RisepelOracle(c2, sd).forward(toks)
        assert row_err(other[window:], want[window:]).max() > 50 * TOL[1]
    with make_engine(cfg, sd, 1) as e:
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[1]          # edges inside one prompt
        assert row_err(replay(e, toks, [window - 1]), want).max() < TOL[1]         # the window fills while decoding
        assert row_err(replay(e, toks, [window + 1, 2, 62]), want).max() < TOL[1]  # edges inside later portions


def test_sink_counts_once_and_first_tokens():
    cfg = ref.random_config(order=("latent_attention",), mlp_on=())
    sd = ref.random_state_dict(cfg, seed=13)
    sd["l0.mix.sink"] = np.asarray([2.0, -1.0, 4.0], np.float32)  # large enough to matter at the first positions
    toks = tokens(5, 12, cfg["vocab"])
    want = ref.RisepelOracle(cfg, sd).forward(toks)
    nosink = dict(sd)
    nosink["l0.mix.sink"] = np.full(3, -60.0, np.float32)
    assert row_err(ref.RisepelOracle(cfg, nosink).forward(toks)[:3], want[:3]).max() > 50 * TOL[1]
    with make_engine(cfg, sd, 1) as e:
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[1]
        assert row_err(replay(e, toks, []), want).max() < TOL[1]


def test_far_token_reaches_through_the_recurrent_state():
    # one early token decides a late logit only through the GLA state: decay close to one, attention window short
    cfg = ref.random_config(order=("gla", "latent_attention"), gla=dict(tau=64.0), lat=dict(window=6))
    sd = ref.random_state_dict(cfg, seed=17)
    a, b = tokens(6, 220, cfg["vocab"]), None
    b = list(a)
    b[3] = (b[3] + 1) % cfg["vocab"]
    o = ref.RisepelOracle(cfg, sd)
    wa, wb = o.forward(a), o.forward(b)
    assert row_err(wb[-1:], wa[-1:]).max() > 10 * TOL[1]  # the far token matters at the end
    with make_engine(cfg, sd, 1) as e:
        assert row_err(replay(e, a, [150, 37]), wa).max() < TOL[1]
        assert row_err(replay(e, b, [5, 2, 130]), wb).max() < TOL[1]


@pytest.mark.parametrize("f32", [1, 0])
def test_long_decoding(f32):
    cfg = ref.random_config()
    sd = ref.random_state_dict(cfg, seed=19)
    toks = tokens(7, 9 + 200, cfg["vocab"])
    want = ref.RisepelOracle(cfg, sd).forward(toks)
    with make_engine(cfg, sd, f32) as e:
        assert row_err(replay(e, toks, [9]), want).max() < TOL[f32]


@pytest.mark.parametrize("f32", [1, 0])
def test_unequal_requests_in_one_batch_match_each_alone(f32):
    cfg = ref.random_config()
    sd = ref.random_state_dict(cfg, seed=23)
    o = ref.RisepelOracle(cfg, sd)
    seqs = [tokens(10 + i, n, cfg["vocab"]) for i, n in enumerate((150, 31, 77, 3))]
    want = [o.forward(t) for t in seqs]
    # per step: how many tokens each sequence advances (0 = sits the step out)
    plan = [(64, 0, 0, 0), (2, 31, 5, 0), (1, 0, 64, 1), (40, 0, 1, 1), (1, 0, 1, 1), (42, 0, 6, 0)]
    with make_engine(cfg, sd, f32) as e:
        solo = [replay(e, t, [len(t)]) for t in seqs]
        ids = [e.seq_open() for _ in seqs]
        at, got = [0] * 4, [[] for _ in seqs]
        for step in plan:
            entries, who = [], []
            for i, n in enumerate(step):
                n = min(n, len(seqs[i]) - at[i])
                if n > 0:
                    entries.append((ids[i], seqs[i][at[i]:at[i] + n], list(range(n))))
                    who.append((i, n))
                    at[i] += n
            out = e.seq_step(entries)
            r = 0
            for i, n in who:
                got[i].append(out[r:r + n])
                r += n
        for sid in ids:
            e.seq_close(sid)
    for i in range(4):
        g = np.concatenate(got[i])
        assert at[i] == len(seqs[i])
        assert row_err(g, want[i]).max() < TOL[f32]
        assert row_err(g, solo[i]).max() < (1e-5 if f32 else 3e-2)


def test_pages_and_slots_are_reused():
    cfg = ref.random_config()
    sd = ref.random_state_dict(cfg, seed=29)
    o = ref.RisepelOracle(cfg, sd)
    with make_engine(cfg, sd, 1, max_seqs=2, ctx=192, pool=256) as e:  # 4 pages, 2 state slots
        total = e.stats()["kv_pages_total"]
        assert total == 4
        for rnd in range(4):  # every round reuses the pages and slots the previous one gave back
            a, b = tokens(40 + rnd, 130, cfg["vocab"]), tokens(50 + rnd, 60, cfg["vocab"])
            sa, sb = e.seq_open(), e.seq_open()
            with pytest.raises(hb.HBError):
                e.seq_open()  # both slots taken
            g1 = e.seq_step([(sa, a[:100], list(range(100))), (sb, b[:33], list(range(33)))])
            g2 = e.seq_step([(sa, a[100:], list(range(30))), (sb, b[33:], list(range(27)))])
            assert e.stats()["kv_pages_free"] == 0  # 3 + 1 pages
            sc_err = None
            try:
                e.seq_step([(sb, [1] * 10, [])])  # would need a fifth page
            except hb.HBError as ex:
                sc_err = ex
            assert sc_err is not None and sc_err.code == -6
            e.seq_close(sa)
            e.seq_close(sb)
            assert e.stats()["kv_pages_free"] == total
            wa, wb = o.forward(a), o.forward(b)
            assert row_err(np.concatenate([g1[:100], g2[:30]]), wa).max() < TOL[1]
            assert row_err(np.concatenate([g1[100:], g2[30:]]), wb).max() < TOL[1]


@pytest.mark.parametrize("f32", [1, 0])
def test_greedy_generation_through_the_scheduler(f32):
    cfg = ref.random_config(vocab=200)
    sd = ref.random_state_dict(cfg, seed=31)
    o = ref.RisepelOracle(cfg, sd)
    prompts = [tokens(60 + i, n, cfg["vocab"]) for i, n in enumerate((70, 5, 129))]
    n_new = 24
    with make_engine(cfg, sd, f32, max_seqs=4, ctx=256) as e:
        rids, outs = e.generate(prompts, hb.Sampling(max_tokens=n_new, capture=CAPTURE_STEP_LOGITS | CAPTURE_PROMPT_LOGITS))
        for p, rid, out in zip(prompts, rids, outs):
            rows = e.captured_logits(rid, CAPTURE_STEP_LOGITS)
            pl = e.captured_logits(rid, CAPTURE_PROMPT_LOGITS)
            assert row_err(pl, o.forward(p)).max() < TOL[f32]
            # teacher-forced comparison of every step's logits; ids must agree wherever the oracle's margin is clear
            st = o.new_state()
            z = o.forward(p, st)[-1]
            for k, t in enumerate(out):
                assert row_err(rows[k][None], z[None]).max() < TOL[f32]
                top2 = np.sort(z)[-2:]
                if top2[1] - top2[0] > 4 * TOL[f32] * np.sqrt((z * z).mean()):
                    assert t == int(np.argmax(z)), (k, t)
                z = o.forward([t], st)[-1]
        assert e.stats()["kv_pages_free"] == e.stats()["kv_pages_total"]


def test_continuous_batching_and_mixed_steps_match_solo_runs():
    cfg = ref.random_config(vocab=200)
    sd = ref.random_state_dict(cfg, seed=37)
    prompts = [tokens(80 + i, n, cfg["vocab"]) for i, n in enumerate((90, 17, 40, 66, 3, 120))]
    sp = hb.Sampling(max_tokens=12)
    with make_engine(cfg, sd, 1, max_seqs=4, ctx=256) as e:
        solo = [e.generate([p], sp)[1][0] for p in prompts]
        _, together = e.generate(prompts, sp)  # more prompts than slots: admission waits for finished sequences
        assert together == solo
    with make_engine(cfg, sd, 1, max_seqs=4, ctx=256, batched=128, decode_with_prefill=1, mixed_step_tokens=64) as e:
        _, mixed = e.generate(prompts, sp)  # prompts cut into 64-token portions beside the running sequences' tokens
        assert e.stats()["steps_mixed"] > 0
        assert mixed == solo
    with make_engine(cfg, sd, 1, max_seqs=4, ctx=256, use_cuda_graphs=1) as e:
        _, graphed = e.generate(prompts, sp)  # decode steps replayed from CUDA graphs (one per batch size)
        assert e.stats()["graph_launches"] > 0
        assert graphed == solo
    with make_engine(cfg, sd, 0, max_seqs=4, ctx=256) as e0, make_engine(cfg, sd, 0, max_seqs=4, ctx=256, use_cuda_graphs=1) as e1:
        assert e0.generate(prompts, sp)[1] == e1.generate(prompts, sp)[1]  # serving mode: same kernels, same ids


def test_random_weights_and_bad_descriptions():
    cfg = ref.random_config()
    sd = ref.random_state_dict(cfg, seed=1)
    desc = weights_io.risepel_desc(cfg, {k: v.shape for k, v in sd.items()})
    with hb.Engine(hb.EngineConfig(device=0, max_seqs=2, max_ctx=128, max_batched_tokens=128)) as e:
        e.load_random(desc, seed=5)
        _, outs = e.generate([tokens(1, 20, cfg["vocab"])], hb.Sampling(max_tokens=4))
        assert len(outs[0]) == 4
    bad = weights_io.risepel_desc(cfg, {k: v.shape for k, v in sd.items()})
    bad.layers[3].kv_from = 2  # a GLA layer holds no cache rows
    with hb.Engine(hb.EngineConfig(device=0, max_seqs=2, max_ctx=128, max_batched_tokens=128)) as e:
        with pytest.raises(hb.HBError):
            e.load_random(bad, seed=5)


def test_tensor_core_head_products_and_long_windows():
    # steps of > 256 tokens with head sizes the tcgen05 GEMM takes: absorption / value expansion per head on the tensor
    # cores, attention of the portion as dense products over a window longer than a query block's own tokens
    cfg = ref.random_config(width=128, order=("latent_attention", "gla", "latent_attention"),
                            lat=dict(heads=2, dim=64, vdim=64, kv_rank=64, q_rank=64, rot_dim=16, window=300), ff=128)
    sd = ref.random_state_dict(cfg, seed=41)
    toks = tokens(8, 700, cfg["vocab"])
    want = ref.RisepelOracle(cfg, sd).forward(toks)
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32, ctx=768) as e:
            assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[f32]
            assert row_err(replay(e, toks, [290, 300, 70, 38]), want).max() < TOL[f32]


def test_window_longer_than_the_context():
    # a window no sequence can fill is full causal attention: nothing may be sized by the configured number
    cfg = ref.random_config(order=("latent_attention", "gla"), lat=dict(window=1 << 20))
    sd = ref.random_state_dict(cfg, seed=43)
    toks = tokens(9, 120, cfg["vocab"])
    want = ref.RisepelOracle(cfg, sd).forward(toks)
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32, ctx=128) as e:
            assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[f32]
            assert row_err(replay(e, toks, [70, 2, 30]), want).max() < TOL[f32]


def test_runtime_serves_a_checkpoint_folder(tmp_path):
    import json
    from helix_b200.runtime import B200Runtime, B200RuntimeParams
    cfg = ref.random_config(vocab=200)
    sd = ref.random_state_dict(cfg, seed=43)
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    weights_io.write_safetensors(tmp_path / "model.safetensors", sd)
    rt = B200Runtime(B200RuntimeParams(model=str(tmp_path), context_length=256, serve_http=False,
                                       args=["--max-num-seqs", "4", "--max-num-batched-tokens", "256"]))
    rt.start()
    try:
        e = rt.engine
        prompt = tokens(9, 50, cfg["vocab"])
        rid = e.submit(prompt, hb.Sampling(max_tokens=8, capture=CAPTURE_STEP_LOGITS))
        out, fin = [], 0
        while not fin:
            assert e.wait(rid, 20000)
            t, fin = e.poll(rid)
            out += t
        rows = e.captured_logits(rid, CAPTURE_STEP_LOGITS)
        o = ref.RisepelOracle(cfg, sd)
        st = o.new_state()
        z = o.forward(prompt, st)[-1]
        for k, t in enumerate(out):  # teacher-forced on the engine's own ids (serving mode)
            assert row_err(rows[k][None], z[None]).max() < TOL[0]
            z = o.forward([t], st)[-1]
        assert len(out) == 8
    finally:
        rt.stop()
