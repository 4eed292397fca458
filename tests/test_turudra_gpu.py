"""Turudra on the GPU against the plain implementation: each mechanism alone, every way of cutting a request, mixed
batches with pages and state slots used again, crafted keys at page borders, long decoding, greedy generation through
the entry point.

Routing note.  In float32 the engine differs from the plain implementation by about 1e-6 of a value's size, so that a
token chooses the same experts unless two router logits tie to that precision; all float32 comparisons are sharp.  In
bfloat16 the router's input differs by about 1e-2, and with random weights a few of some hundred (token, layer) pairs
have two logits that close; such a token takes another expert and its logits move by more than rounding.  The
bfloat16 comparisons against the plain implementation therefore use configurations whose routing has no choice to
make (`top` = experts, one expert), and the one with sparse routing is compared cut against cut (which share their
roundings up to the order of sums) and, against the plain implementation, by the median over positions.
"""
import numpy as np
import pytest
import torch

import plain_turudra as P
import tiny_turudra as tt
import traces

pytestmark = pytest.mark.gpu

LENGTHS = {"mix": [5, 41, 17, 70, 130, 23], "odd": [1, 9, 33, 70, 150, 64], "attn": [3, 29, 66, 100, 129, 48],
           "rec": [2, 19, 90, 35, 60, 77], "tc": [5, 200, 17, 70, 130, 33]}
PAGE = {"mix": 16, "odd": 8, "attn": 64, "rec": 32, "tc": 16}
DENSE = ("odd", "attn", "rec", "tc")          # no routing choice: every expert is chosen


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name in tt.CONFIGS:
        path, cfg, tensors = tt.make_folder(str(tmp_path_factory.mktemp("tu_" + name)), name)
        reqs = {f"r{i}": traces.random_tokens(100 * i + len(name), n, cfg["vocab"]) for i, n in enumerate(LENGTHS[name])}
        ref = {rid: tt.plain_logits(cfg, tensors, t) for rid, t in reqs.items()}
        out[name] = (path, cfg, tensors, reqs, ref)
    return out


def run(folder, dtype, steps, page_size, max_tokens=None, max_requests=4, graphs=True):
    from xyntetik_runner_b200.engine.engine import Engine, EngineParams
    from xyntetik_runner_b200.engine.replay import replay
    mt = max_tokens if max_tokens is not None else traces.pool_tokens(steps, page_size)
    eng = Engine(folder, EngineParams(dtype=dtype, max_tokens=mt, page_size=page_size, max_requests=max_requests, cuda_graphs=graphs))
    res = replay(eng, steps)
    eng.check_status()
    eng.cache.audit()
    assert not eng.cache.live_requests()
    return res, eng


CUTS = {
    "whole": lambda reqs: traces.whole(reqs),
    "tail": lambda reqs: traces.tail_decoded(reqs, 32),
    "portions": lambda reqs: traces.portions(reqs),
    "pairs": lambda reqs: traces.portions(reqs, sizes=(2,)),
    "mixed": lambda reqs: traces.mixed(reqs, seed=3),
    "mixed2": lambda reqs: traces.mixed(reqs, seed=8, max_live=2, sizes=(1, 2, 31, 1, 64, 3)),
}


@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("name", list(tt.CONFIGS))
def test_float32_matches_plain_in_every_cut(models, name, cut):
    path, cfg, tensors, reqs, ref = models[name]
    steps = CUTS[cut](reqs)
    res, eng = run(path, "float32", steps, PAGE[name])
    got = traces.collect(steps, res, cfg["vocab"])
    for rid in reqs:
        traces.assert_close(got[rid], ref[rid], "float32", f"{name}/{cut}/{rid}")
    if cut.startswith("mixed") and eng.cache.pools:
        assert sum(-(-len(t) // PAGE[name]) for t in reqs.values()) > eng.cache.pools[0].n_pages      # pages were used again
    if cut.startswith("mixed"):
        assert len(reqs) > 4            # and so were the state slots


@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("name", DENSE)
def test_bfloat16_matches_plain(models, name, cut):
    path, cfg, tensors, reqs, ref = models[name]
    steps = CUTS[cut](reqs)
    res, _ = run(path, "bfloat16", steps, PAGE[name])
    got = traces.collect(steps, res, cfg["vocab"])
    sharp = 0
    for rid in reqs:
        if tt.recurrence_conditioning(cfg, tensors, reqs[rid]) >= 2.0:
            traces.assert_close(got[rid], ref[rid], "bfloat16", f"{name}/{cut}/{rid}")
            sharp += 1
        else:
            # some token's denominator of the recurrence cancels to within a bfloat16 rounding (see
            # tiny_turudra.recurrence_conditioning): that token may differ; the median position may not
            errs = np.abs(got[rid] - ref[rid]).max(axis=1) / np.abs(ref[rid]).max()
            assert np.median(errs) < 0.5 * traces.TOL["bfloat16"]["max_rel"], (rid, np.median(errs))
    assert sharp >= len(reqs) // 2


def test_bfloat16_sparse_routing_cut_against_cut(models):
    path, cfg, tensors, reqs, ref = models["mix"]
    steps = CUTS["whole"](reqs)
    res, _ = run(path, "bfloat16", steps, PAGE["mix"])
    base = traces.collect(steps, res, cfg["vocab"])
    # against the plain implementation: the median position is within rounding (a few positions may have chosen another expert)
    errs = np.concatenate([np.abs(base[r] - ref[r]).max(axis=1) / np.abs(ref[r]).max() for r in reqs])
    assert np.median(errs) < 0.5 * traces.TOL["bfloat16"]["max_rel"], np.median(errs)      # half of what any position may differ by
    for cut in ("tail", "portions", "mixed", "mixed2"):
        steps = CUTS[cut](reqs)
        res, _ = run(path, "bfloat16", steps, PAGE["mix"])
        got = traces.collect(steps, res, cfg["vocab"])
        errs = np.concatenate([np.abs(got[r] - base[r]).max(axis=1) / np.abs(base[r]).max() for r in reqs])
        # the same products in another tiling: sums in another order, and what that does through a bfloat16 rounding
        assert np.median(errs) < 5e-3 and (errs > 3e-2).mean() < 0.03, (cut, np.median(errs), errs.max())


def test_long_decoding_and_first_tokens(models):
    """Three tokens at once, then 300 one by one: the state is carried 300 times, pages fill and new ones are taken."""
    path, cfg, tensors, _, _ = models["mix"]
    toks = traces.random_tokens(77, 303, cfg["vocab"])
    ref = tt.plain_logits(cfg, tensors, toks)
    steps = traces.tail_decoded({"long": toks}, tail=300)
    res, _ = run(path, "float32", steps, page_size=16, max_tokens=320)
    got = traces.collect(steps, res, cfg["vocab"])["long"]
    traces.assert_close(got, ref, "float32", "long decoding")
    traces.assert_close(got[:3], ref[:3], "float32", "first tokens")


def test_graphs_change_nothing(models):
    path, cfg, tensors, reqs, ref = models["rec"]
    steps = CUTS["tail"](reqs)
    a, _ = run(path, "bfloat16", steps, PAGE["rec"], graphs=True)
    b, _ = run(path, "bfloat16", steps, PAGE["rec"], graphs=False)
    for k in a:
        assert np.array_equal(a[k], b[k])


# ---- mechanisms alone ---------------------------------------------------------------------------------------------
def test_route_topk_kernel():
    from xyntetik_runner_b200 import kernels
    torch.manual_seed(0)
    for E, top in ((16, 4), (5, 5), (1, 1), (70, 3), (33, 32)):
        z = torch.randn(37, E, device="cuda")
        z[3, : min(E, 3)] = 1.5                     # a tie: the lower index first
        ids = torch.empty(37, top, dtype=torch.int32, device="cuda")
        wts = torch.empty(37, top, device="cuda")
        kernels.route_topk(z, ids, wts, top)
        order = sorted(range(E), key=lambda e: (-float(z[3, e]), e))[:top]
        assert ids[3].tolist() == order
        best, idx = torch.topk(z, top, dim=-1)
        assert torch.equal(torch.sort(ids.long(), dim=-1)[0], torch.sort(idx, dim=-1)[0]) or E <= 3
        want = torch.softmax(torch.gather(z, 1, ids.long()), dim=-1)
        assert torch.allclose(wts, want, rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_experts_kernels_against_plain(dtype):
    """Plan, both grouped products and the weighted sum, with more rows per expert than one tile and experts nobody chose."""
    from xyntetik_runner_b200 import kernels
    torch.manual_seed(1)
    n, W, E, top, F, limit = 300, 40, 7, 2, 24, 0.9
    h = torch.randn(n, W).to(dtype)
    wr = torch.randn(E, W)
    wr[5] = -100.0 * h.float().mean(0).sign()      # expert 5 is (almost) never chosen
    wgu = (torch.randn(E, 2 * F, W) / W ** 0.5).to(torch.bfloat16)
    wd = (torch.randn(E, W, F) / F ** 0.5).to(torch.bfloat16)
    z = h.float() @ wr.T
    dev = "cuda"
    ids = torch.empty(n, top, dtype=torch.int32, device=dev)
    wts = torch.empty(n, top, device=dev)
    kernels.route_topk(z.to(dev), ids, wts, top)
    pairs = n * top
    align = kernels.moe_tile_rows()
    max_tiles = kernels.moe_max_tiles(pairs, E, align)
    rows = max_tiles * align
    row_src = torch.empty(rows, dtype=torch.int32, device=dev)
    pair_row = torch.empty(pairs, dtype=torch.int32, device=dev)
    tiles = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    kernels.moe_plan(ids, row_src, pair_row, tiles, E, align)
    assert row_src[pair_row.long()].tolist() == list(range(pairs)) and int((row_src >= 0).sum()) == pairs
    owner = tiles.long().repeat_interleave(align)
    live = row_src >= 0
    assert torch.equal(owner[live], ids.reshape(-1).long()[row_src[live].long()])       # every row lies in a tile of its expert
    assert 5 not in tiles.tolist() or int((ids == 5).sum()) > 0
    y = torch.zeros(rows, F, dtype=dtype, device=dev)
    kernels.moe_gemm(h.to(dev), wgu.to(dev), y, row_src, tiles, top, True, kernels.ACT_SWISH_CLAMP, limit)
    zz = torch.zeros(rows, W, device=dev)
    kernels.moe_gemm(y, wd.to(dev), zz, row_src, tiles, top, False)
    if dtype == torch.bfloat16 and W % 8 == 0 and F % 8 == 0:
        # the same through the tensor-core product over rows sorted by expert, for every row tile it takes
        for bn in (16, 32, 64, 128):
            mt = kernels.moe_max_tiles(pairs, E, bn)
            rs = torch.empty(mt * bn, dtype=torch.int32, device=dev)
            pr = torch.empty(pairs, dtype=torch.int32, device=dev)
            tg = torch.empty(mt, dtype=torch.int32, device=dev)
            kernels.moe_plan(ids, rs, pr, tg, E, bn)
            xs = torch.empty(mt * bn, W, dtype=dtype, device=dev)
            kernels.moe_gather(h.to(dev), xs, rs, tg, top, bn)
            y2 = torch.zeros(mt * bn, F, dtype=dtype, device=dev)
            kernels.gemm_tc_grouped(xs, kernels.pack_weight_groups(wgu.to(dev), 2), y2, tg, bn, F, kernels.EPI_GATED, kernels.ACT_SWISH_CLAMP, limit)
            z2 = torch.zeros(mt * bn, W, device=dev)
            kernels.gemm_tc_grouped(y2, kernels.pack_weight_groups(wd.to(dev)), z2, tg, bn, W)
            kernels.tc_check_status(torch.device(dev))
            a, b2 = z2[pr.long()], zz[pair_row.long()]
            assert (a - b2).abs().max() < 2e-2 * b2.abs().max(), bn
    d = torch.ones(n, W, device=dev)
    kernels.moe_combine(d, zz, wts, pair_row, top)
    want = torch.ones(n, W, dtype=torch.float64)
    hd = h.double()
    for t in range(n):
        for j in range(top):
            e = int(ids[t, j])
            want[t] += float(wts[t, j]) * P.expert(hd[t:t + 1], wgu[e, :F].double(), wgu[e, F:].double(), wd[e].double(), limit)[0]
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (d.cpu().double() - want).abs().max() < tol * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_recurrence_kernel_against_plain(dtype):
    """Two requests of unequal length in one step, from states that an earlier step left, in state slots 2 and 0."""
    from xyntetik_runner_b200 import kernels
    torch.manual_seed(2)
    H, D, V, cap, eps, W = 3, 10, 37, 5.0, 1e-5, 16
    m = {"heads": H, "dim": D, "vdim": V, "gate_cap": cap}
    w = {"q": torch.randn(H * D, W), "k": torch.randn(H * D, W), "v": torch.randn(H * V, W), "g": torch.randn(H * V, W),
         "o": torch.eye(H * V), "norm": torch.rand(H * V) + 0.5, "i": torch.randn(H, W), "i.b": torch.randn(H),
         "f": torch.randn(H, W), "f.b": torch.randn(H) + 2}
    w = {k: v.double() for k, v in w.items()}
    lens, slots = [21, 5], [2, 0]
    hs = [torch.randn(5 + L, W).to(dtype) for L in lens]             # 5 tokens of history each, then this step's
    n = sum(lens)
    state = torch.zeros(4, kernels.mlstm_state_floats(H, D, V), device="cuda")
    want = []
    for h, L, s in zip(hs, lens, slots):
        st = {"S": torch.zeros(H, D, V, dtype=torch.float64), "n": torch.zeros(H, D, dtype=torch.float64), "m": torch.zeros(H, dtype=torch.float64)}
        P.mlstm(h[:5].double(), w, m, eps, st)
        per_head = torch.cat([st["S"].reshape(H, -1), st["n"], st["m"][:, None]], dim=1)
        state[s] = per_head.reshape(-1).float().cuda()
        want.append(P.mlstm(h[5:].double(), w, m, eps, st))
    want = torch.cat(want)
    x = torch.cat([h[5:] for h in hs]).double()
    proj = torch.cat([x @ w[a].T for a in ("q", "k", "v", "g")], dim=1).to(dtype).cuda()
    gates = torch.cat([x @ w["i"].T + w["i.b"], x @ w["f"].T + w["f.b"]], dim=1).float().cuda()
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    coef = torch.empty(n, 3 * H, device="cuda")
    o = torch.empty(n, H * V, device="cuda")
    y = torch.empty(n, H * V, dtype=dtype, device="cuda")
    kernels.mlstm(proj, (0, H * D, 2 * H * D, 2 * H * D + H * V), gates, state, coef, o, w["norm"].float().cuda(), y,
                  i32([0, lens[0]]), i32(lens), i32(slots), 2, H, D, V, cap, eps)
    if dtype == torch.float32:
        assert (y.cpu().double() - want).abs().max() < 2e-5 * want.abs().max()
    else:
        # the plain implementation sees unrounded projections: compare with it fed the rounded ones instead
        assert (y.cpu().double() - want).abs().max() < 5e-2 * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_kernel_reads_the_right_rows(dtype):
    """Rows scattered over pages in no order; for chosen queries one key is made to stand out (the first row, the last
    of a page, the first of the next, one far back, the query's own), and the output must be that row's latent."""
    from xyntetik_runner_b200 import kernels
    torch.manual_seed(3)
    H, C, R, page, n_ctx = 5, 24, 6, 8, 150
    n_pages = 40
    rows = (torch.randn(n_ctx, C + R) * 0.3).to(dtype)
    perm = torch.randperm(n_pages)[: -(-n_ctx // page)].to(torch.int32)
    cache = torch.zeros(n_pages, page, C + R, dtype=dtype)
    for p in range(n_ctx):
        cache[perm[p // page], p % page] = rows[p]
    cases = [(149, 0), (149, 7), (149, 8), (149, 149), (100, 63), (100, 64), (100, 3), (9, 8), (8, 8), (7, 0), (0, 0)]
    n = len(cases)
    ql = torch.randn(n, H, C) * 0.1
    qr = (torch.randn(n, H, R) * 0.1).to(dtype)
    for i, (pos, key) in enumerate(cases):
        ql[i, 2] = rows[key, :C].float() * 60.0          # head 2 of every case looks for `key`
        qr[i, 2] = (rows[key, C:].float() * 60.0).to(dtype)
    dev = "cuda"
    out = torch.empty(n, H * C, device=dev)
    positions = torch.tensor([c[0] for c in cases], dtype=torch.int32, device=dev)
    tok_seg = torch.zeros(n, dtype=torch.int32, device=dev)
    bt = torch.full((1, 32), -1, dtype=torch.int32)
    bt[0, : len(perm)] = perm
    cache_d, qr_d = cache.to(dev), qr.reshape(n, H * R).contiguous().to(dev)
    kernels.latent_attention(ql.reshape(n, H * C).to(dev), qr_d, 0, R, out, cache_d.data_ptr(), page * (C + R), positions, tok_seg,
                             bt.to(dev), H, C, R, 32, page, 1.0)
    out = out.cpu().view(n, H, C)
    for i, (pos, key) in enumerate(cases):
        k = rows[: pos + 1].double()
        q = torch.cat([ql[i].double(), qr[i].double()], dim=1)            # [H, C + R]
        a = torch.softmax(q @ k.T, dim=-1)
        want = a @ k[:, :C]
        assert (out[i].double() - want).abs().max() < 1e-4, (pos, key)
        assert a[2, key] > 0.9 and (out[i, 2].double() - k[key, :C]).abs().max() < 0.1 * k[key, :C].abs().max() + 0.05


def test_latent_attention_on_tensor_cores_against_the_plain_kernel():
    """The same cached rows and queries through both kernels, in one range of keys and in many (some of them empty)."""
    from xyntetik_runner_b200 import kernels
    torch.manual_seed(4)
    dev = "cuda"
    for H, C, R, page, n_ctx in ((5, 64, 8, 8, 150), (20, 128, 16, 16, 300), (16, 512, 64, 64, 700)):
        n_pages = -(-n_ctx // page) + 7
        rows = (torch.randn(n_ctx, C + R) * 0.3).to(torch.bfloat16)
        perm = torch.randperm(n_pages)[: -(-n_ctx // page)].to(torch.int32)
        cache = torch.zeros(n_pages, page, C + R, dtype=torch.bfloat16)
        for p in range(n_ctx):
            cache[perm[p // page], p % page] = rows[p]
        positions = [n_ctx - 1, 0, 31, 32, 33, n_ctx // 2, 127, 128]
        n = len(positions)
        ql = (torch.randn(n, H * C) * 0.2).to(torch.bfloat16).to(dev)
        qr = (torch.randn(n, H * R) * 0.2).to(torch.bfloat16).to(dev)
        ql[0, C:2 * C] = (rows[3, :C].float() * 8).to(torch.bfloat16).to(dev)          # head 1 of the last position looks far back
        pos_d = torch.tensor(positions, dtype=torch.int32, device=dev)
        seg = torch.zeros(n, dtype=torch.int32, device=dev)
        mp = len(perm) + 3
        bt = torch.full((1, mp), -1, dtype=torch.int32)
        bt[0, : len(perm)] = perm
        bt, cache_d = bt.to(dev), cache.to(dev)
        want = torch.empty(n, H * C, device=dev)
        kernels.latent_attention(ql.float(), qr, 0, R, want, cache_d.data_ptr(), page * (C + R), pos_d, seg, bt, H, C, R, mp, page, 0.7)
        mt = -(-H // 16)
        for chunk, splits in ((-(-n_ctx // 32) * 32, 1), (32, -(-n_ctx // 32)), (128, -(-n_ctx // 128) + 2)):
            got = torch.full((n, H * C), float("nan"), device=dev)
            po = torch.full((n * mt * splits * 16 * C,), float("nan"), device=dev)
            pm = torch.full((n * mt * splits * 32,), float("nan"), device=dev)
            kernels.latent_attention_mma(ql, qr, 0, R, got, po, pm, cache_d.data_ptr(), page * (C + R), pos_d, seg, bt, H, C, R, mp,
                                         page, 0.7, chunk, splits)
            err = (got - want).abs().max().item()
            assert err < 1.5e-2 * want.abs().max().item(), (H, C, R, chunk, splits, err)          # P is rounded to bfloat16


def test_far_key_through_the_engine(models):
    """A one-layer attention model whose query and key weights are scaled so that one far key dominates a late query:
    the late position's logits then depend on the far token, across several pages, in a prompt and in decoding."""
    cfg = {"architecture": "Turudra", "vocab": 50, "width": 32, "embedding": {"scale": 1.0}, "residual_mult": 1.0,
           "norm": {"eps": 1e-5}, "logit_softcap": None, "loop": None,
           "layers": [{"type": "latent_attention", "mlp": None,
                       "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 8, "kv_rank": 12, "scale": 4.0, "rot": {"base": 10000.0, "dims": 4}}}]}
    tensors = tt.draw(cfg, 5)
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        path, _, _ = tt.make_folder(tmp, None, tensors, cfg)
        toks = traces.random_tokens(5, 200, 50)
        ref = tt.plain_logits(cfg, tensors, toks)
        other = list(toks)
        other[3] = (toks[3] + 7) % 50                       # change one far token
        ref_other = tt.plain_logits(cfg, tensors, other)
        sharp = np.abs(ref[150:] - ref_other[150:]).max(axis=1)
        assert (sharp > 1e-3).any()                           # the late logits do depend on it
        for steps in (traces.whole({"a": toks}), traces.tail_decoded({"a": toks}, 60), traces.portions({"a": toks}, sizes=(2, 29, 5))):
            res, _ = run(path, "float32", steps, page_size=16)
            traces.assert_close(traces.collect(steps, res, 50)["a"], ref, "float32", "far key")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(models, dtype):
    from xyntetik_runner_b200.engine.runner import Runner
    name = "odd"
    path, cfg, tensors, _, _ = models[name]
    prompts = [traces.random_tokens(i + 40, n, cfg["vocab"]) for i, n in enumerate((5, 11, 17, 3, 30))]
    r = Runner(path, dtype=dtype, ctx=128, parallel=3, page_size=16)          # five requests over three slots
    res = r.generate(prompts, n=12, temp=0.0, ignore_eos=True)
    same = 0
    for p, g in zip(prompts, res):
        assert len(g.tokens) == 12 and g.finish_reason == "length"
        want = tt.plain_greedy(cfg, tensors, p, 12)
        if dtype == "float32":
            assert g.tokens == want
        else:
            # teacher-forced: every token is the plain argmax for the engine's own prefix, or within rounding of it
            for i, tok in enumerate(g.tokens):
                lg = tt.plain_logits(cfg, tensors, list(p) + list(g.tokens[:i]))[-1]
                assert lg.max() - lg[tok] <= 0.06 * np.abs(lg).max()


def test_command_line_generates_what_the_plain_implementation_does(models):
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    path, cfg, tensors, _, _ = models["rec"]
    prompt = traces.random_tokens(9, 7, cfg["vocab"])
    ids = "ids:" + ",".join(str(t) for t in prompt)
    out = {}
    for extra in (["--dtype", "float32"], ["--ref"]):
        r = subprocess.run([sys.executable, os.path.join(root, "bin", "runner"), "-m", path, "-p", ids, "-n", "6", "--ignore-eos"] + extra,
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        out[extra[-1]] = [ln for ln in r.stdout.splitlines() if ln.startswith("ids:")][0]
    want = "ids:" + ",".join(str(t) for t in tt.plain_greedy(cfg, tensors, prompt, 6))
    assert out["--ref"] == want and out["float32"] == want, out
