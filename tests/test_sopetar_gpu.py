"""Sopetar on the GPU against the plain float64 restatement (tests/sopetar_oracle.py): every mechanism alone, whole prompts with the
stream after every layer, decoding through the cache, portions down to two tokens, unequal requests in one batch, pages and slots that are
freed and used again, keys that stand out just inside and just outside the window and the kept first positions (in prompts and in
decoding, at page borders), other sizes (also values that happen to be equal or 1), and greedy generation through the scheduler and
the command lines. Small random models, made here; fp32 mode is compared tightly, bf16 mode within the rounding of bf16 operands."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import sopetar_oracle as O  # noqa: E402
import sopetar_testlib as L  # noqa: E402

pytestmark = pytest.mark.gpu

F32_TOL = 2e-5     # relative rms of a vector, fp32 mode
BF16_TOL = 1e-1    # bf16 operands of the products: worst position
BF16_TYPICAL = 2e-2

CFG_A = L.make_config([L.latent_layer(), L.attention_layer(v_mix=True), L.latent_layer(heads=2, dim=16, rot_dim=8, rot_dims=4, vdim=8, kv_rank=24, size=7, keep_first=2, ff=None),
                       L.attention_layer(heads=6, kv_heads=2, v_mix=True, size=33, keep_first=0, softcap=0), L.attention_layer(heads=2, kv_heads=2, dim=8, vdim=8, size=None)])
# values that a model may happen to make equal or 1: one head, one layer kind, windows of one position and wider than any prompt, no cap,
# no feed-forward, a scale of one on the embedding, a single blending layer (it keeps its values and nobody reads them)
CFG_ONES = L.make_config([L.attention_layer(heads=1, kv_heads=1, dim=32, vdim=32, size=1, keep_first=1, softcap=0, v_mix=True, ff=None),
                          L.latent_layer(heads=1, dim=16, rot_dim=16, vdim=16, kv_rank=16, size=4096)], vocab=61, width=32, embedding_scale=1.0)
# head widths the tensor-core attention takes (multiples of 16 / 8), in both mixers
CFG_TC = L.make_config([L.attention_layer(heads=4, kv_heads=2, dim=32, vdim=16, size=40, keep_first=5, v_mix=True, ff=64),
                        L.latent_layer(heads=4, dim=16, rot_dim=16, vdim=24, kv_rank=48, size=40, ff=64),
                        L.attention_layer(heads=4, kv_heads=2, dim=32, vdim=16, size=70, keep_first=2, v_mix=True, ff=64)], width=64)
# sizes that are multiples of nothing: odd width and vocabulary, head widths that 16-byte loads do not divide, more query heads per
# key/value head than a decoding work item takes, a window larger than the kept positions' reach and one smaller than them
CFG_ODD = L.make_config([L.latent_layer(heads=3, dim=6, rot_dim=10, rot_dims=6, vdim=5, kv_rank=13, size=19, keep_first=25, ff=23),
                         L.attention_layer(heads=34, kv_heads=1, dim=6, vdim=10, size=45, keep_first=50, softcap=3.0, scale=0.7, ff=17),
                         L.attention_layer(heads=3, kv_heads=3, dim=11, vdim=7, size=2, keep_first=1, v_mix=True, ff=None)], vocab=67, width=50, eps=1e-6)


def _engine(tmp_path, cfg, w, dtype="float32", max_tokens=512, max_seqs=4, page_len=32, name="m", **kw):
    from simplellminference_b200.models import build_model
    from simplellminference_b200.seqengine import SequenceEngine
    folder = L.write_model(str(tmp_path / name), cfg, w)
    model = build_model(folder, dtype, "cuda")
    return SequenceEngine(model, max_tokens=max_tokens, max_seqs=max_seqs, page_len=page_len, **kw)


def _logits(eng, slot, toks, want=None):
    want = list(range(len(toks))) if want is None else want
    out = eng.run([(slot, toks, want)])
    return None if out is None else out.cpu().numpy()


def _rel(got, want):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    return float(np.sqrt(((got - want) ** 2).mean()) / max(1e-30, np.sqrt((want ** 2).mean())))


def _w64(w):
    return {k: v.astype(np.float64) for k, v in w.items()}


# ------------------------------------------------------------------------------------------------ mechanisms alone
class _MixersOnly:
    """A model of a few mixers run one after the other on the SAME input rows, which the test hands in; each one's projected output is kept."""

    def __init__(self, groups, width):
        self.groups, self.width = groups, width
        self.h, self.outs = None, None

    def state_specs(self):
        return [g.state_spec() for g in self.groups]

    def forward(self, step, ids, states, rows, n_rows, tap=None):
        self.outs = []
        for g, st in zip(self.groups, states):
            y = step.scratch("sub_out", step.T * self.width)
            g.forward(step, self.h, st, y)
            self.outs.append(y[:step.T * self.width].view(step.T, self.width).clone())
        return None


def _run_mixers(layer_cfgs, w, width, h, portions, dtype="float32", page_len=32, eps=1e-5, blend=False):
    """The mixers of the given layers (each with its output projection, without feed-forward) over h [T][d], fed in portions."""
    import torch

    from simplellminference_b200 import layers
    from simplellminference_b200.config import BF16, F32, SopetarConfig
    from simplellminference_b200.seqengine import SequenceEngine
    from simplellminference_b200.seqops import Ops
    dev = torch.device("cuda")
    ops = Ops(BF16 if dtype == "bfloat16" else F32)
    wt = {k: torch.tensor(v, device=dev, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32) for k, v in w.items()}
    cfg = SopetarConfig.from_dict(L.make_config(layer_cfgs, width=width))
    groups = []
    for i, lc in enumerate(cfg.layers):
        if lc.type == "attention":
            share = None if not blend else ("keep" if i == 0 else "blend")
            mech = layers.CappedWindowAttention(lc.mixer, wt, f"l{i}.mix.", ops, dev, eps, share)
        else:
            mech = layers.LatentAttention(lc.mixer, wt, f"l{i}.mix.", ops, dev, eps)
        groups.append(layers.MixerGroup([("mix", mech, 1.0)], ops, dev))
    stub = _MixersOnly(groups, width)
    stub.ops, stub.device = ops, dev
    eng = SequenceEngine(stub, max_tokens=1024, page_len=page_len, graphs=False)
    slot, outs, p = eng.admit(), [[] for _ in groups], 0
    for n in portions:
        stub.h = torch.tensor(h[p:p + n], dtype=torch.float32, device=dev).contiguous().view(-1)
        eng.run([(slot, np.zeros(n, np.int32), [])])
        for i, o in enumerate(stub.outs):
            outs[i].append(o.cpu().numpy())
        p += n
    return [np.concatenate(o) for o in outs]


ALONE = [L.attention_layer(), L.attention_layer(heads=3, kv_heads=3, dim=20, vdim=36, size=9, keep_first=0, softcap=0),
         L.attention_layer(heads=8, kv_heads=1, dim=8, vdim=8, size=64, keep_first=40, softcap=2.0, scale=1.0), L.attention_layer(size=None),
         L.latent_layer(), L.latent_layer(heads=1, dim=24, rot_dim=4, vdim=70, kv_rank=72, size=33, keep_first=1),
         L.latent_layer(heads=5, dim=4, rot_dim=16, rot_dims=6, vdim=12, kv_rank=20, size=None), L.latent_layer(heads=2, dim=8, rot_dim=8, vdim=8, kv_rank=264, size=50)]


@pytest.mark.parametrize("portions", [[75], [33, 2, 31, 1, 1, 1, 1, 5]])
def test_each_mixer_alone(portions):
    rng = np.random.default_rng(5)
    d, T = 48, 75
    for layer_cfg in ALONE:
        w = L.random_weights(L.make_config([layer_cfg], width=d), seed=11)
        h = rng.standard_normal((T, d)).astype(np.float32)
        got = _run_mixers([layer_cfg], w, d, h, portions)[0]
        if layer_cfg["type"] == "attention":
            want, _ = O.capped_biased_attention(h.astype(np.float64), _w64(w), "l0.mix.", layer_cfg["mixer"], 1e-5)
        else:
            want = O.latent_attention(h.astype(np.float64), _w64(w), "l0.mix.", layer_cfg["mixer"], 1e-5)
        assert _rel(got, want) < F32_TOL, (layer_cfg["mixer"], _rel(got, want))


@pytest.mark.parametrize("portions", [[50], [7, 2, 30, 1, 10]])
def test_values_blended_with_the_first_layers(portions):
    rng = np.random.default_rng(6)
    d, T = 32, 50
    cfgs = [L.attention_layer(heads=2, kv_heads=2, vdim=12, v_mix=True), L.attention_layer(heads=4, kv_heads=2, vdim=12, size=11, v_mix=True)]
    w = L.random_weights(L.make_config(cfgs, width=d), seed=12)
    h = rng.standard_normal((T, d)).astype(np.float32)
    got = _run_mixers(cfgs, w, d, h, portions, blend=True)
    want0, v_first = O.capped_biased_attention(h.astype(np.float64), _w64(w), "l0.mix.", cfgs[0]["mixer"], 1e-5)
    want1, _ = O.capped_biased_attention(h.astype(np.float64), _w64(w), "l1.mix.", cfgs[1]["mixer"], 1e-5, v_first)
    plain1, _ = O.capped_biased_attention(h.astype(np.float64), _w64(w), "l1.mix.", cfgs[1]["mixer"], 1e-5)
    assert _rel(want1, plain1) > 1e-2, "the blend does not show in this test's numbers"
    assert _rel(got[0], want0) < F32_TOL and _rel(got[1], want1) < F32_TOL


def _standing_out(kind, d, H, window, keep_first):
    """A one-mixer layer and weights in which the query of a position reads the first third of its input row and the key the second
    third, through the same map: a query row whose first third repeats the second third of an earlier row gives that position (and no
    other, itself included) a score far above the rest. Returns (layer, weights, third)."""
    t = d // 3
    if kind == "attention":
        layer = L.attention_layer(heads=H, kv_heads=H, dim=16, vdim=16, scale=4.0, softcap=200.0, size=window, keep_first=keep_first)
        w = L.random_weights(L.make_config([layer], width=d), seed=3)
        a = w["l0.mix.q"][:, :t].copy()
        w["l0.mix.q"][:] = 0.0
        w["l0.mix.k"][:] = 0.0
        w["l0.mix.q"][:, :t] = a
        w["l0.mix.k"][:, t:2 * t] = a
        w["l0.mix.k.b"] = w["l0.mix.q.b"].copy()
        w["l0.mix.v"][:, :2 * t] = 0.0
    else:
        R, dn = 32, 16
        layer = L.latent_layer(heads=H, dim=dn, rot_dim=4, vdim=16, kv_rank=R, scale=1.0, size=window, keep_first=keep_first)
        w = L.random_weights(L.make_config([layer], width=d), seed=3)
        # the latent reads the second third through m; head h's unrotated query is W_uk,h m applied to the FIRST third:
        # q_h(row i) . k_h(row j) = |W_uk,h m x|^2 / rms(m x) when row i's first third and row j's second third are both x
        m = w["l0.mix.dkv"][:R, t:2 * t].astype(np.float64)
        w["l0.mix.dkv"][:R] = 0.0
        w["l0.mix.dkv"][:R, t:2 * t] = m
        q = np.zeros((H, dn + 4, d), np.float32)
        uk = w["l0.mix.uk"].reshape(H, dn, R).astype(np.float64)
        for hd in range(H):
            q[hd, :dn, :t] = L.bf16_round(3.0 * uk[hd] @ m)
        w["l0.mix.q"] = q.reshape(H * (dn + 4), d)
        w["l0.mix.dkv.norm"] = np.ones(R, np.float32)
        w["l0.mix.sink"] = np.zeros(H, np.float32)
    return layer, w, t


@pytest.mark.parametrize("kind", ["attention", "latent"])
@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decoded"])
def test_keys_just_inside_and_outside_the_window_and_the_kept_first_positions(kind, decode):
    """The key input of an earlier position is repeated as the query input of a later one: when that position is visible (the oldest one inside the window, or
    the last of the kept first positions) the query's output is essentially its value, when it is one further (just outside the window, the
    first position that is not kept) the output is something else — the restatement says so and the engine has to follow it in both cases,
    with the key's page before, at and after a page border."""
    rng = np.random.default_rng(9)
    d, T, H, window, keep = 48, 150, 2, 37, 3
    layer, w, t = _standing_out(kind, d, H, window, keep)
    fn = (lambda h: O.capped_biased_attention(h, _w64(w), "l0.mix.", layer["mixer"], 1e-5)[0]) if kind == "attention" else \
         (lambda h: O.latent_attention(h, _w64(w), "l0.mix.", layer["mixer"], 1e-5))
    seen_diff = []
    for query in (149, 100, 68, 69, 70):                      # oldest visible key 113 / 64 / 32 / 33 / 34: around the borders of pages of 32
        for key, visible in ((query - window + 1, True), (query - window, False), (keep - 1, True), (keep, False)):
            h = rng.standard_normal((T, d)).astype(np.float32)
            h[query, :t] = h[key, t:2 * t]
            want = fn(h.astype(np.float64))
            portions = [query] + [1] * (T - query) if decode else [T]
            got = _run_mixers([layer], w, d, h, portions)[0]
            assert _rel(got, want) < F32_TOL, (kind, query, key, _rel(got, want))
            base = h.copy()
            base[key] = rng.standard_normal(d)
            seen_diff.append((visible, _rel(fn(base.astype(np.float64))[query], want[query])))
    shown = sorted(r for v, r in seen_diff if v)
    assert shown[0] > 0.05 and shown[len(shown) // 2] > 0.5, "a visible repeated position does not stand out: the test would not notice a lost key"
    assert max(r for v, r in seen_diff if not v) < 1e-6, "a hidden position changes the restatement's result"


def test_row_kernels():
    import torch

    from simplellminference_b200.config import F32
    from simplellminference_b200.seqops import Ops
    ops, dev, rng = Ops(F32), torch.device("cuda"), np.random.default_rng(2)
    st = torch.cuda.current_stream().cuda_stream
    for T, d in ((5, 48), (3, 1000), (2, 4100)):
        x = (rng.standard_normal((T, d)) * 3 + 1.5).astype(np.float32)
        wv, bv = rng.standard_normal(d).astype(np.float32), rng.standard_normal(d).astype(np.float32)
        xt, y = torch.tensor(x, device=dev), torch.empty(T, d, device=dev)
        ops.layernorm(xt, d, torch.tensor(wv, device=dev), torch.tensor(bv, device=dev), 1e-5, y, d, T, d, st)
        assert _rel(y.cpu().numpy(), O.layer_norm(x.astype(np.float64), wv, bv, 1e-5)) < 1e-6
        # depth average: planes [x | hist 0 .. n_prev]
        n_prev = 3
        hist = rng.standard_normal((n_prev + 1, T, d)).astype(np.float32)
        yv, coef = rng.standard_normal((T, d)).astype(np.float32), rng.standard_normal(n_prev + 1).astype(np.float32)
        ht, h_out = torch.tensor(hist, device=dev), torch.empty(T, d, device=dev)
        ops.depth_average(xt, torch.tensor(yv, device=dev), ht, n_prev, torch.tensor(coef, device=dev), torch.tensor(wv, device=dev), torch.tensor(bv, device=dev),
                          1e-5, h_out, T, d, st)
        own = x.astype(np.float64) + yv
        mixed = sum(coef[j] * hist[j].astype(np.float64) for j in range(n_prev)) + coef[n_prev] * own
        assert _rel(ht[n_prev].cpu().numpy(), own) < 1e-6 and _rel(xt.cpu().numpy(), mixed) < 1e-6
        assert _rel(h_out.cpu().numpy(), O.layer_norm(mixed, wv, bv, 1e-5)) < 2e-6
        # the feed-forward's activation on columns of a wider matrix
        n = d // 2
        z = (rng.standard_normal((T, d)) * 2).astype(np.float32)
        zt, out = torch.tensor(z, device=dev), torch.empty(T, n, device=dev)
        ops.clamped_glu(zt.data_ptr(), d, zt.data_ptr() + 4 * n, d, 1.25, 1.702, out, n, T, n, st)
        g, u = np.minimum(z[:, :n].astype(np.float64), 1.25), np.clip(z[:, n:2 * n].astype(np.float64), -1.25, 1.25)
        assert _rel(out.cpu().numpy(), g * O.sigmoid(1.702 * g) * (u + 1)) < 1e-6
    torch.cuda.synchronize()


def test_feed_forward_alone():
    """The clamped feed-forward through MixerGroup (fused gate / up product, activation, down projection with bias)."""
    import torch

    from simplellminference_b200 import layers
    from simplellminference_b200.config import F32, SopetarConfig
    from simplellminference_b200.seqengine import SequenceEngine
    from simplellminference_b200.seqops import Ops
    rng, d, T = np.random.default_rng(4), 40, 21
    cfg = L.make_config([L.latent_layer(ff=56, limit=0.75)], width=d)
    w = L.random_weights(cfg, seed=2)
    dev, ops = torch.device("cuda"), Ops(F32)
    wt = {k: torch.tensor(v, device=dev) for k, v in w.items()}
    ff = layers.ClampedGluFeedForward(SopetarConfig.from_dict(cfg).layers[0].mlp, wt, "l0.mlp.", ops, dev)
    stub = _MixersOnly([layers.MixerGroup([("ff", ff, 1.0)], ops, dev)], d)
    stub.ops, stub.device = ops, dev
    eng = SequenceEngine(stub, max_tokens=64, graphs=False)
    h = (2 * rng.standard_normal((T, d))).astype(np.float32)
    stub.h = torch.tensor(h, device=dev).view(-1)
    eng.run([(eng.admit(), np.zeros(T, np.int32), [])])
    assert _rel(stub.outs[0].cpu().numpy(), O.clamped_glu(h.astype(np.float64), _w64(w), "l0.mlp.", cfg["layers"][0]["mlp"])) < F32_TOL


# ------------------------------------------------------------------------------------------------ whole models
@pytest.mark.parametrize("cfg", [CFG_A, CFG_ONES, CFG_TC, CFG_ODD], ids=["mixed", "ones", "tensorcore", "odd"])
def test_whole_prompt_matches_oracle_fp32_and_layers(tmp_path, cfg):
    w = L.random_weights(cfg, seed=1)
    toks = np.random.default_rng(2).integers(0, cfg["vocab"], size=140).tolist()
    taps_want = []
    want = O.forward(cfg, _w64(w), toks, taps_want)
    eng = _engine(tmp_path, cfg, w)
    taps = []
    got = eng.run([(eng.admit(), toks, list(range(len(toks))))], tap=lambda i, x: taps.append(x.clone().cpu().numpy())).cpu().numpy()
    assert len(taps) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(taps, taps_want)):
        assert _rel(a, b) < F32_TOL, (i, _rel(a, b))
    assert L.logit_error(got, want).max() < F32_TOL


@pytest.mark.parametrize("cfg", [CFG_A, CFG_TC, CFG_ODD], ids=["mixed", "tensorcore", "odd"])
def test_bf16_mode_within_operand_rounding(tmp_path, cfg):
    w = L.random_weights(cfg, seed=3)
    toks = np.random.default_rng(4).integers(0, cfg["vocab"], size=150).tolist()
    want = O.forward(cfg, _w64(w), toks)
    eng = _engine(tmp_path, cfg, w, dtype="bfloat16")
    s = eng.admit()
    whole = _logits(eng, s, toks)
    eng.release(s)
    s = eng.admit()
    cut = np.concatenate([_logits(eng, s, toks[:100]), _logits(eng, s, toks[100:102])] + [_logits(eng, s, toks[p:p + 1]) for p in range(102, 150)])
    for got in (whole, cut):
        e = L.logit_error(got, want)
        assert e.max() < BF16_TOL and np.median(e) < BF16_TYPICAL, (e.max(), np.median(e))


@pytest.mark.parametrize("cfg", [CFG_A, CFG_ONES, CFG_TC, CFG_ODD], ids=["mixed", "ones", "tensorcore", "odd"])
def test_prefill_against_token_by_token_and_portions(tmp_path, cfg):
    w = L.random_weights(cfg, seed=5)
    toks = np.random.default_rng(6).integers(0, cfg["vocab"], size=120).tolist()
    want = O.forward(cfg, _w64(w), toks)
    eng = _engine(tmp_path, cfg, w)
    for portions in ([1] * 120, [2] * 60, [31, 2, 33, 1, 1, 40, 12], [64, 56], [119, 1]):
        s, outs, p = eng.admit(), [], 0
        for n in portions:
            outs.append(_logits(eng, s, toks[p:p + n]))
            p += n
        eng.release(s)
        assert L.logit_error(np.concatenate(outs), want).max() < F32_TOL, portions[:3]


def test_unequal_requests_in_one_batch_and_reuse_of_pages_and_slots(tmp_path):
    """Seven requests of unequal length through three slots and ten pages of 32: portions of prompts beside single tokens of others, every
    request's logits equal the restatement's of that request alone; pages and slots go from finished requests to new ones."""
    cfg = CFG_A
    w = L.random_weights(cfg, seed=7)
    rng = np.random.default_rng(8)
    lens = [70, 33, 5, 96, 64, 1, 47]
    reqs = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lens]
    want = [O.forward(cfg, _w64(w), r) for r in reqs]
    eng = _engine(tmp_path, cfg, w, max_tokens=320, max_seqs=3, page_len=32)
    waiting, slots, fed, got = list(range(len(reqs))), {}, [0] * len(reqs), [[] for _ in reqs]
    used_slots, page_users, step = [], {}, 0
    sizes = [17, 2, 32, 5, 40, 3]
    while waiting or slots:
        while waiting and len(slots) < 3 and eng.free_pages >= -(-lens[waiting[0]] // 32) + sum(-(-lens[i] // 32) - eng.pages.held(s) for i, s in slots.items()):
            i = waiting.pop(0)
            slots[i] = eng.admit()
            used_slots.append(slots[i])
        entries, order = [], []
        for i, s in slots.items():
            left = lens[i] - fed[i]
            n = 1 if (fed[i] > lens[i] // 2) else min(left, sizes[(step + i) % len(sizes)])   # portions first, single tokens later
            entries.append((s, reqs[i][fed[i]:fed[i] + n], list(range(n))))
            order.append((i, n))
        out = eng.run(entries).cpu().numpy()
        table = eng.pages.table()
        for i, sl in slots.items():
            for pg in table[sl]:
                if pg >= 0:
                    page_users.setdefault(int(pg), set()).add(i)
        r = 0
        for i, n in order:
            got[i].append(out[r:r + n])
            r += n
            fed[i] += n
        for i in [i for i in slots if fed[i] == lens[i]]:
            eng.release(slots.pop(i))
        step += 1
    assert len(used_slots) > len(set(used_slots)), "no slot was used twice: the test does not test reuse"
    assert eng.free_pages == 10 and any(len(u) > 1 for u in page_users.values()), "no page went from one request to another"
    for i in range(len(reqs)):
        assert L.logit_error(np.concatenate(got[i]), want[i]).max() < F32_TOL, i


def test_long_decoding_over_page_borders_and_past_the_window(tmp_path):
    cfg = L.make_config([L.attention_layer(size=50, keep_first=4, v_mix=True), L.latent_layer(size=70), L.attention_layer(size=130, keep_first=0, v_mix=True)])
    w = L.random_weights(cfg, seed=8)
    toks = np.random.default_rng(4).integers(0, cfg["vocab"], size=330).tolist()
    want = O.forward(cfg, _w64(w), toks)
    eng = _engine(tmp_path, cfg, w, max_tokens=384, page_len=64)
    s = eng.admit()
    outs = [_logits(eng, s, toks[:60])] + [_logits(eng, s, toks[p:p + 1]) for p in range(60, 330)]
    assert eng.graph_replays > 200
    assert L.logit_error(np.concatenate(outs), want).max() < F32_TOL


def test_first_tokens_of_a_sequence_after_a_used_slot(tmp_path):
    """A slot and pages that held a long request serve the next one: its first tokens equal the restatement's."""
    w = L.random_weights(CFG_A, seed=9)
    rng = np.random.default_rng(10)
    eng = _engine(tmp_path, CFG_A, w, max_seqs=1, max_tokens=96)
    for n in (90, 4, 1, 2, 35):
        toks = rng.integers(0, CFG_A["vocab"], size=n).tolist()
        s = eng.admit()
        got = _logits(eng, s, toks)
        eng.release(s)
        assert L.logit_error(got, O.forward(CFG_A, _w64(w), toks)).max() < F32_TOL, n


def _follows_greedy(cfg, w, prompt, produced):
    seq = list(prompt)
    for k, tok in enumerate(produced):
        lg = O.forward(cfg, _w64(w), seq)[-1]
        order = np.argsort(lg)
        close = lg[order[-1]] - lg[order[-2]] <= 1e-3 * np.abs(lg).max()      # a near tie may fall either way: follow the engine
        assert tok == int(order[-1]) or (close and tok == int(order[-2])), (prompt[:4], k)
        seq.append(tok)


def test_greedy_generation_through_the_scheduler(tmp_path):
    """Requests of unequal length through ContinuousBatcher over SequenceDecoder (prompts in portions beside decoding requests, more
    requests than slots): every request's tokens are the restatement's greedy continuation of that prompt alone."""
    from simplellminference_b200.scheduler import ContinuousBatcher
    from simplellminference_b200.seqengine import SequenceDecoder
    cfg = CFG_A
    w = L.random_weights(cfg, seed=12)
    rng = np.random.default_rng(13)
    prompts = [rng.integers(0, cfg["vocab"], size=n).tolist() for n in (5, 40, 1, 23, 64, 7)]
    new = 10
    eng = _engine(tmp_path, cfg, w, max_tokens=6 * 32, max_seqs=3, page_len=32)
    cb = ContinuousBatcher(SequenceDecoder(eng, prefill_chunk=16), chunk=4)
    ids = [cb.submit(p, new) for p in prompts]
    out = cb.run()
    assert cb.stats.max_live == 3 and eng.free_pages == 6
    for rid, p in zip(ids, prompts):
        got = [int(t) for t in out[rid]]
        assert got[:len(p) - 1] == p[1:]
        _follows_greedy(cfg, w, p, got[len(p) - 1:])


def test_trace_replayer_command(tmp_path):
    """bin/trace_run end to end on a Sopetar folder: the model class comes from config.json."""
    import json
    import subprocess
    cfg = CFG_ONES
    w = L.random_weights(cfg, seed=15)
    folder = L.write_model(str(tmp_path / "model"), cfg, w)
    rng = np.random.default_rng(16)
    a, b = rng.integers(0, cfg["vocab"], size=70).tolist(), rng.integers(0, cfg["vocab"], size=9).tolist()
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b, "want": [8]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[31:], "want": [38]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "c", "tokens": b, "want": [0, 8]}], "end": ["c"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out_dir = tmp_path / "out"
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", str(out_dir), "--max-tokens", "128"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2", "done 3"]
        wa, wb = O.forward(cfg, _w64(w), a), O.forward(cfg, _w64(w), b)
        V = cfg["vocab"]
        got = [np.fromfile(out_dir / f"{n}.f32", dtype="<f4").reshape(-1, V) for n in range(4)]
        assert L.logit_error(got[0], wa[[0, 29]]).max() < tol and L.logit_error(got[1], np.stack([wa[30], wb[8]])).max() < tol
        assert L.logit_error(got[2], wa[[69]]).max() < tol and L.logit_error(got[3], wb[[0, 8]]).max() < tol


def test_generation_command_line(tmp_path):
    """python -m simplellminference_b200.generate on a Sopetar folder: registry, engine, scheduler, device arg-max."""
    import json
    import subprocess
    cfg = CFG_TC
    w = L.random_weights(cfg, seed=21)
    folder = L.write_model(str(tmp_path / "model"), cfg, w)
    prompts = [[3, 1, 4, 1, 5, 9, 2, 6], [7]]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "simplellminference_b200.generate", "--model", folder, "--dtype", "float32", "--max-new-tokens", "6", "--prefill-chunk", "3"]
    for p in prompts:
        cmd += ["--prompt", ",".join(str(t) for t in p)]
    r = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(ln) for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert [ln["prompt"] for ln in lines] == prompts
    for ln in lines:
        assert len(ln["tokens"]) == 6
        _follows_greedy(cfg, w, ln["prompt"], ln["tokens"])
