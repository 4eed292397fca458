"""Besolix without a GPU: the configuration reader, the plan the builder makes (cache entries that are shared, how long
rows are kept, a norm weight nothing reads), and the plain implementation's own consistency (each mechanism written a
second way)."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_besolix as P
import tiny_besolix as tb
from xyntetik_runner_b200 import architectures  # noqa: F401
from xyntetik_runner_b200.config import registry
from xyntetik_runner_b200.config.base import ConfigError
from xyntetik_runner_b200.config.besolix import BesolixConfig


@pytest.mark.parametrize("name", list(tb.CONFIGS))
def test_config_round_trip_and_tensor_names(name):
    cfg = BesolixConfig.from_dict(tb.CONFIGS[name])
    assert BesolixConfig.from_dict(cfg.to_dict()) == cfg
    plan = registry.resolve("Besolix").build_plan(cfg)
    plan.validate()
    specs = {n: tuple(s.shape) for n, s in plan.tensor_specs().items() if not s.optional}
    assert specs == {n: tuple(s) for n, s in tb.shapes(tb.CONFIGS[name]).items()}
    assert [e.layer for e in plan.schedule] == list(range(len(cfg.layers)))


def test_folder_is_resolved_by_its_architecture_key(tmp_path):
    path, cfg, _ = tb.make_folder(str(tmp_path / "m"), "rec")
    arch, typed = registry.load_config(path)
    assert arch.name == "Besolix" and typed.width == cfg["width"] and len(typed.layers) == 2


@pytest.mark.parametrize("edit, word", [
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda d: d["layers"][0]["mixer"].pop("heads"), "heads"),
    (lambda d: d["layers"][0]["mixer"].__setitem__("kv_heads", 3), "kv_heads"),
    (lambda d: d["layers"][0]["mixer"].pop("conv"), "conv"),
    (lambda d: d["layers"][1]["mixer"].pop("q_rank"), "q_rank"),
    (lambda d: d["layers"][1]["mixer"]["mask"].__setitem__("size", 0), "mask"),
    (lambda d: d["layers"][2]["mixer"]["rot"].__setitem__("dims", 7), "dims"),
    (lambda d: d["layers"][2]["mixer"]["rot"].__setitem__("dims", 26), "dims"),
    (lambda d: d["layers"][3]["mixer"].__setitem__("kv_from", 3), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].__setitem__("kv_from", 2), "kv_from"),
    (lambda d: d["layers"][3]["mixer"].__setitem__("kv_rank", 48), "kv_rank"),
    (lambda d: d["layers"][0]["mlp"].__setitem__("kind", "moe"), "kind"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["norm"].pop("eps"), "eps"),
])
def test_config_refusals(edit, word):
    d = copy.deepcopy(tb.CONFIGS["mix"])
    edit(d)
    with pytest.raises(ConfigError, match=word):
        BesolixConfig.from_dict(d)


def test_a_reader_of_a_readers_rows_is_refused():
    d = copy.deepcopy(tb.CONFIGS["tc"])
    d["layers"][5]["mixer"]["kv_from"] = 3
    with pytest.raises(ConfigError, match="kv_from"):
        BesolixConfig.from_dict(d)


def test_a_reader_may_leave_what_it_shares_to_the_owner():
    d = copy.deepcopy(tb.CONFIGS["mix"])
    for key in ("kv_rank", "rot_dim", "rot"):
        d["layers"][3]["mixer"].pop(key)
    assert BesolixConfig.from_dict(d) == BesolixConfig.from_dict(tb.CONFIGS["mix"])


def test_shared_rows_are_kept_for_the_longest_window_among_their_readers():
    plan = registry.resolve("Besolix").build_plan(BesolixConfig.from_dict(tb.CONFIGS["mix"]))
    assert plan.schedule[3].cache_from == 1 and plan.schedule[1].cache_from is None
    owner, reader = plan.blocks[1].mixer, plan.blocks[3].mixer
    assert (owner.window, reader.window) == (19, 37) and owner.kv_need().window == 37
    assert owner.own_rows and not reader.own_rows
    plan = registry.resolve("Besolix").build_plan(BesolixConfig.from_dict(tb.CONFIGS["tc"]))
    assert plan.blocks[0].mixer.kv_need().window is None          # one of the two readers sees every row
    plan = registry.resolve("Besolix").build_plan(BesolixConfig.from_dict(tb.CONFIGS["win"]))
    assert plan.blocks[1].mixer.kv_need().window == 3


def test_a_second_norm_weight_of_a_layer_without_feed_forward_may_be_there_or_not(tmp_path):
    from xyntetik_runner_b200.weights.loader import FolderSource, WeightsError, load_tensors
    cfg = tb.CONFIGS["rec"]
    plan = registry.resolve("Besolix").build_plan(BesolixConfig.from_dict(cfg))
    specs = plan.tensor_specs()
    assert specs["l0.norm2"].optional and "l1.norm2" in specs and not specs["l1.norm2"].optional
    tensors = tb.draw(cfg, 3)
    path, _, _ = tb.make_folder(str(tmp_path / "without"), None, tensors, cfg)
    got = load_tensors(specs, FolderSource(path), torch.device("cpu"))
    assert "l0.norm2" not in got and "l1.norm2" in got
    tensors["l0.norm2"] = torch.zeros(cfg["width"], dtype=torch.bfloat16)
    path, _, _ = tb.make_folder(str(tmp_path / "with"), None, tensors, cfg)
    assert "l0.norm2" in load_tensors(specs, FolderSource(path), torch.device("cpu"))
    del tensors["l1.norm2"]
    path, _, _ = tb.make_folder(str(tmp_path / "lacking"), None, tensors, cfg)
    with pytest.raises(WeightsError, match="l1.norm2"):
        load_tensors(specs, FolderSource(path), torch.device("cpu"))


# ---- the plain implementation, each mechanism a second way ---------------------------------------------------------
def test_window_mask_edges():
    m = P.window_mask(9, 3)
    assert m[5].tolist() == [False, False, False, True, True, True, False, False, False]
    assert m[1].tolist() == [True, True] + [False] * 7
    assert P.window_mask(4, 1).tolist() == torch.eye(4, dtype=torch.bool).tolist()
    assert P.window_mask(5, None).tolist() == torch.ones(5, 5, dtype=torch.bool).tril().tolist()
    assert P.window_mask(5, 99).tolist() == P.window_mask(5, None).tolist()


def test_rotation_depends_on_the_distance_alone():
    torch.manual_seed(0)
    q, k = torch.randn(1, 12, dtype=torch.float64), torch.randn(1, 12, dtype=torch.float64)

    def score(pq, pk):
        a = P.rotate_adjacent(q, torch.tensor([pq]), 8, 50.0, 2.0)
        b = P.rotate_adjacent(k, torch.tensor([pk]), 8, 50.0, 2.0)
        return float((a * b).sum())
    assert abs(score(40, 33) - score(7, 0)) < 1e-12 and abs(score(40, 33) - score(40, 32)) > 1e-6
    a = P.rotate_adjacent(q, torch.tensor([5]), 8, 50.0)
    assert torch.equal(a[:, 8:], q[:, 8:]) and abs(float(a.norm() - q.norm())) < 1e-12
    # pair (2i, 2i + 1) by hand, scaled frequency
    ang = 5 * 50.0 ** (-2.0 * 1 / 8) / 2.0
    b = P.rotate_adjacent(q, torch.tensor([5]), 8, 50.0, 2.0)
    assert abs(float(b[0, 2]) - (float(q[0, 2]) * math.cos(ang) - float(q[0, 3]) * math.sin(ang))) < 1e-12
    assert abs(float(b[0, 3]) - (float(q[0, 3]) * math.cos(ang) + float(q[0, 2]) * math.sin(ang))) < 1e-12


def test_short_convolution_against_a_loop():
    torch.manual_seed(1)
    z, taps = torch.randn(9, 5, dtype=torch.float64), torch.randn(5, 4, dtype=torch.float64)
    got = P.short_conv(z, taps)
    for t in range(9):
        for c in range(5):
            want = sum(float(taps[c, 3 - j]) * float(z[t - j, c]) for j in range(4) if t - j >= 0)
            assert abs(float(got[t, c]) - want) < 1e-12
    assert torch.allclose(P.short_conv(z, taps[:, -1:]), z * taps[:, -1])


def _delta_weights(W, H, G, D, V, K):
    w = {"q": torch.randn(G * D, W), "k": torch.randn(G * D, W), "v": torch.randn(H * V, W), "g": torch.randn(H * V, W),
         "o": torch.randn(W, H * V), "norm": torch.rand(V) + 0.5, "b": torch.randn(H, W), "a": torch.randn(H, W),
         "A_log": torch.randn(H) - 1, "dt_bias": torch.randn(H), "q.conv": torch.randn(G * D, K), "k.conv": torch.randn(G * D, K),
         "v.conv": torch.randn(H * V, K)}
    return {k: v.double() for k, v in w.items()}


def test_delta_rule_written_with_explicit_matrices():
    """S' = g S (I ... ) form: S_t = g_t (I - beta_t k_t k_t^T) S_{t-1} + beta_t k_t v_t^T, o_t = S_t^T q_t."""
    torch.manual_seed(2)
    W, H, G, D, V, K = 14, 4, 2, 5, 3, 3
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "conv": K}
    w = _delta_weights(W, H, G, D, V, K)
    h = torch.randn(11, W, dtype=torch.float64)
    w_id = dict(w)
    w_id["o"] = torch.eye(H * V, dtype=torch.float64)
    got = P.delta(h, w_id, m, 1e-5).view(11, H, V)
    silu = torch.nn.functional.silu
    q = silu(P.short_conv(h @ w["q"].T, w["q.conv"])).view(11, G, D)
    k = silu(P.short_conv(h @ w["k"].T, w["k.conv"])).view(11, G, D)
    v = silu(P.short_conv(h @ w["v"].T, w["v.conv"])).view(11, H, V)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) / math.sqrt(D)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    gate = silu(h @ w["g"].T).view(11, H, V)
    for hd in range(H):
        kv = hd // (H // G)
        S = torch.zeros(D, V, dtype=torch.float64)
        for t in range(11):
            beta = torch.sigmoid(h[t] @ w["b"][hd])
            g = torch.exp(-torch.exp(w["A_log"][hd]) * torch.log1p(torch.exp(h[t] @ w["a"][hd] + w["dt_bias"][hd])))
            kk = k[t, kv]
            S = g * (torch.eye(D, dtype=torch.float64) - beta * torch.outer(kk, kk)) @ S + beta * torch.outer(kk, v[t, hd])
            o = S.T @ q[t, kv]
            o = o / torch.sqrt((o * o).mean() + 1e-5) * w["norm"] * gate[t, hd]
            assert torch.allclose(o, got[t, hd], atol=1e-10), (hd, t)


def test_latent_attention_with_the_query_taken_into_the_latent_space():
    """(q . W_uk c) = (W_uk^T q) . c and sum a W_uv c = W_uv sum a c: what lets a layer cache the latent alone."""
    torch.manual_seed(3)
    W, H, D, R, V, C, Q, T = 20, 3, 4, 6, 5, 7, 9, 13
    m = {"heads": H, "dim": D, "rot_dim": R, "vdim": V, "kv_rank": C, "q_rank": Q, "scale": 0.4, "rot": {"base": 30.0, "dims": R},
         "mask": {"size": 5}}
    w = {"dq": torch.randn(Q, W), "dq.norm": torch.rand(Q) + 0.5, "uq": torch.randn(H * (D + R), Q), "dkv": torch.randn(C + R, W),
         "dkv.norm": torch.rand(C) + 0.5, "uk": torch.randn(H * D, C), "uv": torch.randn(H * V, C), "g": torch.randn(H * V, W),
         "o": torch.eye(H * V)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, W, dtype=torch.float64)
    got = P.latent_attention(h, w, m, 1e-5).view(T, H, V)
    latent, k_rot = P.latent_rows(h, w, m, 1e-5)
    q = (P.norm_plain(h @ w["dq"].T, w["dq.norm"], 1e-5) @ w["uq"].T).view(T, H, D + R)
    q_rot = P.rotate_adjacent(q[..., D:], torch.arange(T), R, 30.0)
    gate = torch.sigmoid(h @ w["g"].T).view(T, H, V)
    for i in range(T):
        for hd in range(H):
            ql = w["uk"].view(H, D, C)[hd].T @ q[i, hd, :D]
            js = [j for j in range(T) if 0 <= i - j < 5]
            s = torch.stack([(ql @ latent[j] + q_rot[i, hd] @ k_rot[j]) * 0.4 for j in js])
            a = torch.softmax(s, dim=0)
            o = w["uv"].view(H, V, C)[hd] @ sum(a[n] * latent[j] for n, j in enumerate(js))
            assert torch.allclose(o * gate[i, hd], got[i, hd], atol=1e-10)


def test_attention_with_a_window_as_a_loop_over_keys():
    torch.manual_seed(4)
    W, H, G, D, V, T = 16, 4, 2, 6, 3, 12
    m = {"heads": H, "kv_heads": G, "dim": D, "vdim": V, "scale": 0.5, "rot": {"base": 20.0, "dims": 4, "scaling": {"factor": 3.0}},
         "mask": {"size": 4}}
    w = {"q": torch.randn(H * D, W), "k": torch.randn(G * D, W), "v": torch.randn(G * V, W), "q.norm": torch.rand(D) + 0.5,
         "k.norm": torch.rand(D) + 0.5, "o": torch.eye(H * V)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(T, W, dtype=torch.float64)
    got = P.attention(h, w, m, 1e-5).view(T, H, V)
    pos = torch.arange(T)
    q = P.rotate_adjacent(P.norm_plain((h @ w["q"].T).view(T, H, D), w["q.norm"], 1e-5), pos, 4, 20.0, 3.0)
    k = P.rotate_adjacent(P.norm_plain((h @ w["k"].T).view(T, G, D), w["k.norm"], 1e-5), pos, 4, 20.0, 3.0)
    v = (h @ w["v"].T).view(T, G, V)
    for i in range(T):
        for hd in range(H):
            js = list(range(max(0, i - 3), i + 1))
            a = torch.softmax(torch.stack([q[i, hd] @ k[j, hd // 2] * 0.5 for j in js]), dim=0)
            assert torch.allclose(sum(a[n] * v[j, hd // 2] for n, j in enumerate(js)), got[i, hd], atol=1e-10)
    wide = dict(m)
    wide["mask"] = {"size": T}
    none = {k: v for k, v in m.items() if k != "mask"}
    assert torch.allclose(P.attention(h, w, wide, 1e-5), P.attention(h, w, none, 1e-5))


def test_the_norms_and_the_activation():
    x = torch.tensor([[3.0, -4.0]], dtype=torch.float64)
    w = torch.tensor([0.5, -0.25], dtype=torch.float64)
    r = math.sqrt(12.5 + 1e-3)
    assert torch.allclose(P.norm_plain(x, w, 1e-3), torch.tensor([[1.5 / r, 1.0 / r]], dtype=torch.float64))
    assert torch.allclose(P.norm_one_plus(x, w, 1e-3), torch.tensor([[4.5 / r, -3.0 / r]], dtype=torch.float64))
    z = torch.tensor([-2.0, 0.0, 0.7], dtype=torch.float64)
    want = [0.5 * t * (1 + math.tanh(math.sqrt(2 / math.pi) * (t + 0.044715 * t ** 3))) for t in z.tolist()]
    assert torch.allclose(P.gelu_tanh(z), torch.tensor(want, dtype=torch.float64))


def test_a_far_token_reaches_a_late_position_through_the_recurrence_but_not_through_a_window():
    cfg = tb.CONFIGS["win"]
    tensors = tb.draw(cfg, 5)
    toks = [int(t) for t in np.random.RandomState(0).randint(0, cfg["vocab"], size=40)]
    other = list(toks)
    other[2] = (toks[2] + 1) % cfg["vocab"]
    a, b = tb.plain_logits(cfg, tensors, toks), tb.plain_logits(cfg, tensors, other)
    assert np.abs(a[2] - b[2]).max() > 1e-3 and np.abs(a[30:] - b[30:]).max() < 1e-9        # four layers of windows <= 3
    cfg = tb.CONFIGS["rec"]
    tensors = tb.draw(cfg, 5, slow_decay=True)
    toks77 = [t % cfg["vocab"] for t in toks]
    other77 = list(toks77)
    other77[2] = (toks77[2] + 1) % cfg["vocab"]
    a, b = tb.plain_logits(cfg, tensors, toks77), tb.plain_logits(cfg, tensors, other77)
    assert np.abs(a[39] - b[39]).max() > 1e-4
