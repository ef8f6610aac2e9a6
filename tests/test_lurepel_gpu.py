"""Lurepel layer-list decoders through the engine (driven sequences and the scheduler) against the float64 oracle.

Every test builds its own small configuration and random bf16-representable weights (oracle/lurepel_ref.py); the engine
runs them in its exact mode (fp32 weights, cache and products), where a block edge that is one token off, a missing unit in
the softmax denominator or a wrong expert must show, and in its serving mode (bf16 weights / cache rows / GEMM operands)
with a rounding-sized bound.
"""
import copy

import numpy as np
import pytest

import helix_b200 as hb
from helix_b200 import weights_io
from helix_b200.engine import CAPTURE_PROMPT_LOGITS, CAPTURE_STEP_LOGITS, ATTN_UNIT_SINK
from oracle import lurepel_ref as ref
from oracle.weights import to_bf16_f32

pytestmark = pytest.mark.gpu

TOL = {1: 2e-4, 0: 6e-2}  # compute_f32 -> bound on rms(diff) / rms(expected) per logits row


def row_err(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    d = got - want
    return np.sqrt((d * d).mean(-1)) / np.sqrt((want * want).mean(-1))


def oracle_rows(cfg, sd, toks, f32):
    """Expected logits and the rows a comparison may rest on.  A router's choice between two outputs whose choice scores
    nearly tie flips under rounding (serving mode: about 1e-2 of a score), and the flipped token then differs for every
    later token that sees it, which the block mask confines to its own block.  Such rows are left out; the exact mode keeps
    practically all rows and is the sharp test."""
    margins = []
    want = ref.LurepelOracle(cfg, sd).forward(toks, margins=margins)
    ok = np.ones(len(toks), bool)
    if margins:
        sizes = {(ly["mixer"].get("mask") or {}).get("size") or 0 for ly in cfg["layers"]}
        size = sizes.pop() if len(sizes) == 1 else 0
        for t in np.nonzero(np.min(margins, axis=0) < (1e-5 if f32 else 3e-2))[0]:
            ok[t:(t // size + 1) * size if size else len(toks)] = False
    return want, ok


def check(got, want, ok, f32, least=0.15):
    err = row_err(got, want)
    assert ok.mean() >= least, ok.mean()   # the comparison still covers a fair share of the rows
    assert not ok.any() or err[ok].max() < TOL[f32], (err[ok].max(), int(np.argmax(np.where(ok, err, 0))))
    assert err.max() < 1.5                  # a flipped choice changes one unit's output, not the model


def make_engine(cfg, sd, f32, max_seqs=4, ctx=512, pool=0, batched=0, edit=None, **kw):
    desc = weights_io.desc_from_hf_config(copy.deepcopy(cfg), {k: v.shape for k, v in sd.items()}, compute_f32=bool(f32))
    if edit:
        edit(desc)
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
    "default": dict(),
    "attention_alone": dict(order=(None,)),
    "dense_alone": dict(order=("dense",)),
    "moe_alone": dict(order=("moe",)),
    "one_kv_head": dict(heads=4, kv_heads=1),
    "no_grouping": dict(heads=3, kv_heads=3, order=("moe", "dense")),
    "five_heads_per_kv_head": dict(heads=10, kv_heads=2, dim=16, rot_dims=16),  # more than one block's group of query heads
    # nothing a multiple of 8 or 4: every product takes the CUDA-core GEMM, rows are loaded element by element
    "odd_sizes": dict(width=90, vocab=131, heads=6, kv_heads=3, dim=14, rot_dims=6, chunk=9, ff=50, expert_ff=30),
    "no_rotation_causal": dict(rot_dims=0, chunk=0, order=("dense", None)),
    "full_rotation_unscaled": dict(rot_dims=24, scaling=None, base=100.0),
    "scaling_low_not_one": dict(scaling=dict(factor=3.0, low=2.0, high=5.0, original=100), eps=1e-3, scale=0.31),
    "top_one_no_identity": dict(order=("moe", "moe"), identity=0, top=1, experts=3),
    "every_output_chosen": dict(order=("moe",), identity=1, top=4, experts=3),
    "one_expert_many_identities": dict(order=("moe",), identity=3, top=2, experts=1),
    "many_experts": dict(order=("moe", "dense"), experts=70, identity=2, top=5, expert_ff=24),  # router wider than one MMA tile
    "layers_differ": dict(order=("moe", "dense", "moe"), per_layer={0: dict(heads=2, kv_heads=1, dim=40, mask=dict(size=7)),
                                                                    2: dict(heads=8, kv_heads=4, dim=8, rot=dict(base=30.0, dims=4))}),
    # head sizes of the fused tensor-core attention with blocks shorter than its 64-key tiles / longer than a page
    "fused_attention_small_blocks": dict(width=128, heads=4, kv_heads=1, dim=64, rot_dims=64, chunk=20, order=("dense",)),
    "fused_attention_128": dict(width=128, vocab=256, heads=2, kv_heads=2, dim=128, rot_dims=32, chunk=70, order=("dense", None)),
    # inner sizes that are multiples of 128: gate / up rows stored as [128 gate | 128 up] tiles, gated epilogue of the GEMM
    "packed_gated_units": dict(width=128, vocab=256, heads=4, kv_heads=2, dim=64, rot_dims=32, chunk=96, ff=256, expert_ff=128),
    "widest_heads": dict(width=64, heads=2, kv_heads=1, dim=512, rot_dims=128, chunk=33, order=(None,), scale=0.05),
    "tensor_core_shapes": dict(width=128, vocab=256, heads=4, kv_heads=2, dim=64, rot_dims=32, chunk=96, ff=128, expert_ff=64),
}


@pytest.mark.parametrize("f32", [1, 0])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_oracle(name, f32):
    cfg = ref.random_config(**CONFIGS[name])
    sd = ref.random_state_dict(cfg, seed=3)
    toks = tokens(1, 150, cfg["vocab"])  # crosses two page borders and several blocks of every configuration above
    want, ok = oracle_rows(cfg, sd, toks, f32)
    with make_engine(cfg, sd, f32) as e:
        got = replay(e, toks, [len(toks)])
    check(got, want, ok, f32, least=0.0 if name == "layers_differ" else 0.15)


@pytest.mark.parametrize("name", ["tensor_core_shapes", "packed_gated_units"])
def test_steps_of_hundreds_of_tokens_take_the_tensor_core_products(name):
    cfg = ref.random_config(**CONFIGS[name])
    sd = ref.random_state_dict(cfg, seed=5)
    toks = tokens(2, 420, cfg["vocab"])
    for f32 in (1, 0):
        want, ok = oracle_rows(cfg, sd, toks, f32)
        with make_engine(cfg, sd, f32) as e:
            check(replay(e, toks, [len(toks)]), want, ok, f32, least=0.1)
            check(replay(e, toks, [300, 2, 97, 2]), want, ok, f32, least=0.1)


@pytest.mark.parametrize("f32", [1, 0])
def test_prefill_portions_and_single_tokens_agree(f32):
    cfg = ref.random_config()
    sd = ref.random_state_dict(cfg, seed=7)
    toks = tokens(3, 140, cfg["vocab"])
    want, ok = oracle_rows(cfg, sd, toks, f32)
    with make_engine(cfg, sd, f32) as e:
        whole = replay(e, toks, [len(toks)])
        for cuts in ([64, 64], [63, 2, 2, 61], [19, 20, 21, 2, 45], [1, 1, 1, 2, 3, 64, 5], []):
            got = replay(e, toks, cuts)
            check(got, want, ok, f32)
            # the same positions, cut differently: rounding only
            assert row_err(got, whole)[ok].max() < (1e-5 if f32 else 3e-2), cuts


def sharpen(cfg, factor):
    """Peaked softmax: single keys dominate, so a key wrongly seen or missed moves the logits by far more than rounding."""
    cfg = copy.deepcopy(cfg)
    for ly in cfg["layers"]:
        ly["mixer"]["scale"] *= factor
    return cfg


@pytest.mark.parametrize("chunk", [5, 63, 64, 65, 70])
def test_block_edges_in_prompts_and_decoding(chunk):
    cfg = sharpen(ref.random_config(order=(None,), chunk=chunk), 3.0)
    sd = ref.random_state_dict(cfg, seed=11)
    toks = tokens(4, 2 * chunk + 64 + 9, cfg["vocab"])
    want = ref.LurepelOracle(cfg, sd).forward(toks)
    # a block that is one position longer / shorter, or blocks counted from another origin, are far away
    for dc in (-1, 1):
        other = ref.LurepelOracle(sharpen(ref.random_config(order=(None,), chunk=chunk + dc), 3.0), sd).forward(toks)
        assert row_err(other[chunk:], want[chunk:]).max() > 50 * TOL[1]
    with make_engine(cfg, sd, 1) as e:
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[1]             # edges inside one prompt
        assert row_err(replay(e, toks, [chunk - 1]), want).max() < TOL[1]             # the block ends while decoding
        assert row_err(replay(e, toks, [chunk + 1, 2, chunk - 2, 3]), want).max() < TOL[1]  # portions that start inside a block
        assert row_err(replay(e, toks, [chunk, chunk]), want).max() < TOL[1]          # portions that are whole blocks
    with make_engine(cfg, sd, 0) as e:
        assert row_err(replay(e, toks, [chunk + 1, 2, chunk - 2, 3]), want).max() < TOL[0]


def test_first_tokens_and_the_unit_in_the_denominator():
    cfg = ref.random_config(order=(None,), chunk=8)
    sd = ref.random_state_dict(cfg, seed=13)
    toks = tokens(5, 20, cfg["vocab"])
    want = ref.LurepelOracle(cfg, sd).forward(toks)
    without = copy.deepcopy(cfg)
    without["layers"][0]["mixer"]["sink"] = False
    bare = ref.LurepelOracle(without, sd).forward(toks)
    # the first position of every block sees one key: without the unit its weight would be exactly one
    assert row_err(bare[[0, 8, 16]], want[[0, 8, 16]]).min() > 50 * TOL[1]
    with make_engine(cfg, sd, 1) as e:
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[1]
        assert row_err(replay(e, toks, []), want).max() < TOL[1]

    def no_sink(desc):
        for l in desc.layers:
            l.attn_flags &= ~ATTN_UNIT_SINK
    with make_engine(cfg, sd, 1, edit=no_sink) as e:  # the flag is a parameter of the mechanism
        assert row_err(replay(e, toks, [7, 2]), bare).max() < TOL[1]


def test_values_are_raw_keys_and_gate_reads_the_layer_input():
    # the two places where a plausible other reading exists: values taken after the rotation / normalisation, and a gate
    # applied per channel or from the attention output.  The oracle states the design; here its alternatives must differ.
    cfg = ref.random_config(order=(None,))
    sd = ref.random_state_dict(cfg, seed=17)
    toks = tokens(6, 40, cfg["vocab"])
    o = ref.LurepelOracle(cfg, sd)
    want = o.forward(toks)
    m, p = cfg["layers"][0]["mixer"], o.P["layers"][0]["mix"]
    x = ref.norm_gain(o.P["embed"][np.asarray(toks)], o.P["embed_norm"], o.eps)
    kn, v = ref.attention_kv(x, p, m, np.arange(len(toks)), o.eps)
    assert np.abs(kn - v).max() > 0.1                                      # normalised keys are not the values
    assert np.allclose(v.reshape(len(toks), -1), x @ p["k"].T)            # the values are the projection itself
    with make_engine(cfg, sd, 1) as e:
        assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[1]


def test_far_keys_and_page_borders():
    # one block of 300 positions: the last positions look back over four pages; with a peaked softmax the keys that win are
    # anywhere in it.  The same tokens under blocks of 128 differ wherever a far key mattered.
    cfg = sharpen(ref.random_config(order=("dense",), chunk=300, heads=4, kv_heads=2), 4.0)
    sd = ref.random_state_dict(cfg, seed=19)
    toks = tokens(7, 290, cfg["vocab"])
    # plant one far key: position 3's token returns at the end, so the last query finds its own key direction 286 back
    toks[-1] = toks[3]
    want = ref.LurepelOracle(cfg, sd).forward(toks)
    near = ref.LurepelOracle(sharpen(ref.random_config(order=("dense",), chunk=128, heads=4, kv_heads=2), 4.0), sd).forward(toks)
    assert row_err(near[260:], want[260:]).max() > 50 * TOL[1]
    for f32 in (1, 0):
        with make_engine(cfg, sd, f32) as e:
            assert row_err(replay(e, toks, [len(toks)]), want).max() < TOL[f32]
            assert row_err(replay(e, toks, [255, 2, 1, 1, 1, 2]), want).max() < TOL[f32]  # decoding over the page border at 256


@pytest.mark.parametrize("shape", [dict(dim=64, heads=6, kv_heads=2, chunk=70), dict(dim=128, heads=8, kv_heads=1, chunk=150),
                                   dict(dim=64, heads=2, kv_heads=2, chunk=0)])
def test_single_token_steps_on_the_tensor_core_decode_kernel(shape):
    # serving mode, head sizes of the TMA decode kernel: block starts inside its 128-key tiles, blocks that end while decoding,
    # one to three sequences per step at different depths (one split per CTA up to sixteen)
    cfg = ref.random_config(width=128, vocab=256, rot_dims=32, order=("dense", None), **shape)
    sd = ref.random_state_dict(cfg, seed=59)
    o = ref.LurepelOracle(cfg, sd)
    seqs = [tokens(70 + i, n, cfg["vocab"]) for i, n in enumerate((330, 200, 150))]
    want = [o.forward(s) for s in seqs]
    with make_engine(cfg, sd, 0, ctx=384) as e:
        assert row_err(replay(e, seqs[0], [5]), want[0]).max() < TOL[0]  # 325 single-token steps of one sequence
        ids = [e.seq_open() for _ in seqs]
        starts = (130, 3, 64)
        for i, sid in enumerate(ids):
            e.seq_step([(sid, seqs[i][:starts[i]], [])])
        got, at = [[] for _ in seqs], list(starts)
        while any(at[i] < len(seqs[i]) for i in range(3)):
            live = [i for i in range(3) if at[i] < len(seqs[i])]
            out = e.seq_step([(ids[i], [seqs[i][at[i]]], [0]) for i in live])
            for r, i in enumerate(live):
                got[i].append(out[r])
                at[i] += 1
        for i in range(3):
            assert row_err(np.stack(got[i]), want[i][starts[i]:]).max() < TOL[0]


def test_long_decoding_over_blocks_and_pages():
    cfg = ref.random_config(chunk=50)
    sd = ref.random_state_dict(cfg, seed=23)
    toks = tokens(8, 230, cfg["vocab"])
    want, ok = oracle_rows(cfg, sd, toks, 1)
    with make_engine(cfg, sd, 1) as e:
        check(replay(e, toks, [10]), want, ok, 1)  # 220 single-token steps
    want, ok = oracle_rows(cfg, sd, toks, 0)
    with make_engine(cfg, sd, 0, use_cuda_graphs=1) as e:
        check(replay(e, toks, [10]), want, ok, 0)


def test_router_choice_weights_and_identity_outputs():
    # the router alone, on inputs made for it: corrections that change the choice but not the weights, identity outputs
    cfg = ref.random_config(order=("moe",), experts=4, identity=2, top=2)
    sd = ref.random_state_dict(cfg, seed=29)
    corr = np.array(sd["l0.mlp.correction"], np.float32)
    corr[5] = 4.0   # an identity output is always chosen ...
    corr[0] = -4.0  # ... and expert 0 never
    sd["l0.mlp.correction"] = corr
    toks = tokens(9, 60, cfg["vocab"])
    o = ref.LurepelOracle(cfg, sd)
    want = o.forward(toks)
    x = np.random.default_rng(0).standard_normal((16, cfg["width"]))
    idx, wt = ref.moe_route(x, o.P["layers"][0]["mlp"], cfg["layers"][0]["mlp"]["router"])
    assert (idx[:, 0] == 5).all() and (idx != 0).all() and (wt < 1.0).all() and (wt.sum(-1) < 1.0).all()
    plain = dict(sd)
    plain["l0.mlp.correction"] = np.zeros(6, np.float32)
    assert row_err(ref.LurepelOracle(cfg, plain).forward(toks), want).max() > 50 * TOL[1]
    for f32 in (1, 0):
        _, ok = oracle_rows(cfg, sd, toks, f32)
        with make_engine(cfg, sd, f32) as e:
            check(replay(e, toks, [33, 2]), want, ok, f32)


@pytest.mark.parametrize("f32", [1, 0])
def test_mixed_batches_match_each_request_alone(f32):
    cfg = ref.random_config()
    sd = ref.random_state_dict(cfg, seed=31)
    o = ref.LurepelOracle(cfg, sd)
    seqs = [tokens(20 + i, n, cfg["vocab"]) for i, n in enumerate((150, 37, 90, 64))]
    want, oks = zip(*[oracle_rows(cfg, sd, s, f32) for s in seqs])
    plans = [[64, 2, 30, 1, 1, 1, 51], [1, 1, 1, 1, 1, 1, 31], [3, 64, 2, 1, 20], [2, 2, 2, 2, 56]]
    with make_engine(cfg, sd, f32) as e:
        solo = [replay(e, s, p) for s, p in zip(seqs, plans)]
        ids = [e.seq_open() for _ in seqs]
        at, got = [0] * 4, [[] for _ in seqs]
        plans = [list(p) for p in plans]
        step = 0
        while any(at[i] < len(seqs[i]) for i in range(4)):
            entries, who = [], []
            for i in range(4):
                if at[i] >= len(seqs[i]) or (step + i) % 5 == 4:  # every request sits out some steps
                    continue
                n = min(plans[i].pop(0) if plans[i] else 1, len(seqs[i]) - at[i])
                entries.append((ids[i], seqs[i][at[i]:at[i] + n], list(range(n))))
                who.append((i, n))
                at[i] += n
            step += 1
            if not entries:
                continue
            out, r = e.seq_step(entries), 0
            for i, n in who:
                got[i].append(out[r:r + n])
                r += n
        for sid in ids:
            e.seq_close(sid)
    for i in range(4):
        g = np.concatenate(got[i])
        check(g, want[i], oks[i], f32)
        assert row_err(g, solo[i])[oks[i]].max() < (1e-5 if f32 else 3e-2)


def test_pages_and_slots_are_reused():
    cfg = ref.random_config()
    sd = ref.random_state_dict(cfg, seed=37)
    o = ref.LurepelOracle(cfg, sd)
    with make_engine(cfg, sd, 1, max_seqs=2, ctx=192, pool=256) as e:  # 4 pages, 2 sequences
        total = e.stats()["kv_pages_total"]
        assert total == 4
        for rnd in range(4):  # every round reuses the pages and slots the previous one gave back
            a, b = tokens(40 + rnd, 130, cfg["vocab"]), tokens(50 + rnd, 60, cfg["vocab"])
            sa, sb = e.seq_open(), e.seq_open()
            with pytest.raises(hb.HBError):
                e.seq_open()
            g1 = e.seq_step([(sa, a[:100], list(range(100))), (sb, b[:33], list(range(33)))])
            g2 = e.seq_step([(sa, a[100:], list(range(30))), (sb, b[33:], list(range(27)))])
            assert e.stats()["kv_pages_free"] == 0  # 3 + 1 pages
            e.seq_close(sa)
            e.seq_close(sb)
            assert e.stats()["kv_pages_free"] == total
            wa, wb = o.forward(a), o.forward(b)
            assert row_err(np.concatenate([g1[:100], g2[:30]]), wa).max() < TOL[1]
            assert row_err(np.concatenate([g1[100:], g2[30:]]), wb).max() < TOL[1]


@pytest.mark.parametrize("f32", [1, 0])
def test_greedy_generation_through_the_scheduler(f32):
    # serving mode without routers: a choice that flips under rounding would change every later token of the sequence
    cfg = ref.random_config(vocab=200) if f32 else ref.random_config(vocab=200, order=("dense", None, "dense"))
    sd = ref.random_state_dict(cfg, seed=41)
    o = ref.LurepelOracle(cfg, sd)
    prompts = [tokens(60 + i, n, cfg["vocab"]) for i, n in enumerate((70, 5, 129))]
    with make_engine(cfg, sd, f32, max_seqs=4, ctx=256) as e:
        rids, outs = e.generate(prompts, hb.Sampling(max_tokens=24, capture=CAPTURE_STEP_LOGITS | CAPTURE_PROMPT_LOGITS))
        for p, rid, out in zip(prompts, rids, outs):
            rows = e.captured_logits(rid, CAPTURE_STEP_LOGITS)
            assert row_err(e.captured_logits(rid, CAPTURE_PROMPT_LOGITS), o.forward(p)).max() < TOL[f32]
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
    sd = ref.random_state_dict(cfg, seed=43)
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


def test_block_longer_than_the_context_and_random_weights():
    # a block no sequence can fill is causal attention: nothing may be sized by the configured number
    cfg = ref.random_config(chunk=1 << 20)
    sd = ref.random_state_dict(cfg, seed=47)
    toks = tokens(9, 120, cfg["vocab"])
    for f32 in (1, 0):
        want, ok = oracle_rows(cfg, sd, toks, f32)
        with make_engine(cfg, sd, f32, ctx=128) as e:
            check(replay(e, toks, [70, 2, 30]), want, ok, f32, least=0.1)
    desc = weights_io.desc_from_hf_config(cfg)
    with hb.Engine(hb.EngineConfig(device=0, max_seqs=2, max_ctx=128, max_batched_tokens=128)) as e:
        e.load_random(desc, seed=5)
        _, outs = e.generate([tokens(1, 20, cfg["vocab"])], hb.Sampling(max_tokens=4))
        assert len(outs[0]) == 4
    desc.layers[0].kv_heads = 4  # 6 query heads do not split over 4
    with hb.Engine(hb.EngineConfig(device=0, max_seqs=2, max_ctx=128, max_batched_tokens=128)) as e:
        with pytest.raises(hb.HBError):
            e.load_random(desc, seed=5)


def test_runtime_serves_a_checkpoint_folder(tmp_path):
    import json
    from helix_b200.runtime import B200Runtime, B200RuntimeParams
    cfg = ref.random_config(vocab=200, order=("dense", None, "dense"))
    sd = ref.random_state_dict(cfg, seed=53)
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
        o = ref.LurepelOracle(cfg, sd)
        st = o.new_state()
        z = o.forward(prompt, st)[-1]
        for k, t in enumerate(out):  # teacher-forced on the engine's own ids (serving mode)
            assert row_err(rows[k][None], z[None]).max() < TOL[0]
            z = o.forward([t], st)[-1]
        assert len(out) == 8
    finally:
        rt.stop()
