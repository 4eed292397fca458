"""Turudra without a GPU: the configuration reader, the plan the builder makes, and the plain implementation's own
consistency (a recurrence carried over a cut equals the whole; attention written as a loop over keys)."""
import copy

import numpy as np
import pytest
import torch

import plain_turudra as P
import tiny_turudra as tt
from xyntetik_runner_b200 import architectures  # noqa: F401
from xyntetik_runner_b200.config import registry
from xyntetik_runner_b200.config.base import ConfigError
from xyntetik_runner_b200.config.turudra import TurudraConfig


@pytest.mark.parametrize("name", list(tt.CONFIGS))
def test_config_round_trip_and_tensor_names(name):
    cfg = TurudraConfig.from_dict(tt.CONFIGS[name])
    assert TurudraConfig.from_dict(cfg.to_dict()) == cfg
    plan = registry.resolve("Turudra").build_plan(cfg)
    specs = plan.tensor_specs()
    want = tt.shapes(tt.CONFIGS[name])
    assert {n: tuple(s.shape) for n, s in specs.items()} == {n: tuple(s) for n, s in want.items()}
    runs = [(e.layer, e.before is not None) for e in plan.schedule]
    assert runs == P.layer_order(tt.CONFIGS[name])
    plan.validate()


def test_folder_is_resolved_by_its_architecture_key(tmp_path):
    path, cfg, _ = tt.make_folder(str(tmp_path / "m"), "rec")
    arch, typed = registry.load_config(path)
    assert arch.name == "Turudra" and typed.width == cfg["width"] and len(typed.layers) == 2


@pytest.mark.parametrize("edit, word", [
    (lambda d: d["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda d: d["layers"][0]["mixer"].pop("heads"), "heads"),
    (lambda d: d["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda d: d["loop"].__setitem__("stop", 99), "loop"),
    (lambda d: d.pop("width"), "width"),
    (lambda d: d["norm"].pop("eps"), "eps"),
    (lambda d: d["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "dims"),
])
def test_config_refusals(edit, word):
    d = copy.deepcopy(tt.CONFIGS["mix"])
    edit(d)
    with pytest.raises(ConfigError, match=word):
        TurudraConfig.from_dict(d)


def test_plain_recurrence_carries_over_a_cut():
    torch.manual_seed(0)
    m = {"heads": 2, "dim": 6, "vdim": 10, "gate_cap": 7.0}
    W = 20
    w = {"q": torch.randn(12, W), "k": torch.randn(12, W), "v": torch.randn(20, W), "g": torch.randn(20, W),
         "o": torch.randn(W, 20), "norm": torch.rand(20) + 0.5, "i": torch.randn(2, W), "i.b": torch.randn(2),
         "f": torch.randn(2, W), "f.b": torch.randn(2) + 2}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(17, W, dtype=torch.float64)
    whole = P.mlstm(h, w, m, 1e-5)
    st = None
    parts = []
    for a, b in ((0, 1), (1, 3), (3, 11), (11, 17)):
        st = st or {"S": torch.zeros(2, 6, 10, dtype=torch.float64), "n": torch.zeros(2, 6, dtype=torch.float64),
                    "m": torch.zeros(2, dtype=torch.float64)}
        parts.append(P.mlstm(h[a:b], w, m, 1e-5, st))
    assert torch.allclose(torch.cat(parts), whole, rtol=1e-12, atol=1e-12)


def test_plain_recurrence_first_token_by_hand():
    """One token, one head: m1 = max(lf, li) because the running maximum starts at 0, not at minus infinity."""
    m = {"heads": 1, "dim": 2, "vdim": 2, "gate_cap": 100.0}
    W = 2
    eye = torch.eye(2, dtype=torch.float64)
    w = {"q": eye, "k": eye, "v": eye, "g": torch.zeros(2, 2, dtype=torch.float64), "o": eye,
         "norm": torch.ones(2, dtype=torch.float64), "i": torch.zeros(1, 2, dtype=torch.float64),
         "i.b": torch.tensor([-3.0], dtype=torch.float64), "f": torch.zeros(1, 2, dtype=torch.float64),
         "f.b": torch.tensor([0.0], dtype=torch.float64)}
    h = torch.tensor([[1.0, 2.0]], dtype=torch.float64)
    li = 100 * np.tanh(-3 / 100)
    lf = np.log(0.5)
    m1 = max(lf + 0.0, li)
    i1 = np.exp(li - m1)
    q = np.array([1.0, 2.0]) / np.sqrt(2)
    S = i1 * np.outer([1.0, 2.0], [1.0, 2.0])
    n = i1 * np.array([1.0, 2.0])
    o = S.T @ q / (max(abs(n @ q), np.exp(-m1)) + 1e-6)
    o = o / np.sqrt((o * o).mean() + 1e-5) * 0.5
    got = P.mlstm(h, w, m, 1e-5)[0].numpy()
    assert np.allclose(got, o, rtol=1e-12)


def test_plain_attention_as_a_loop_over_keys():
    torch.manual_seed(1)
    m = {"heads": 2, "dim": 4, "rot_dim": 4, "vdim": 3, "kv_rank": 5, "scale": 0.3, "rot": {"base": 50.0, "dims": 4}}
    W = 12
    w = {"q": torch.randn(16, W), "dkv": torch.randn(9, W), "dkv.norm": torch.rand(5) + 0.5, "uk": torch.randn(8, 5),
         "uv": torch.randn(6, 5), "g": torch.randn(2, W), "o": torch.randn(W, 6)}
    w = {k: v.double() for k, v in w.items()}
    h = torch.randn(6, W, dtype=torch.float64)
    got = P.latent_attention(h, w, m, 1e-5)
    # by hand for the last token
    T = 6
    down = h @ w["dkv"].T
    c = down[:, :5] / torch.sqrt((down[:, :5] ** 2).mean(-1, keepdim=True) + 1e-5) * w["dkv.norm"]

    def rot(v, p):
        f = torch.tensor([50.0 ** 0.0, 50.0 ** -0.5], dtype=torch.float64)
        a = p * f
        return torch.cat([v[:2] * torch.cos(a) - v[2:] * torch.sin(a), v[2:] * torch.cos(a) + v[:2] * torch.sin(a)])
    out = []
    q = (h[T - 1] @ w["q"].T).view(2, 8)
    for hd in range(2):
        s = []
        for j in range(T):
            k_plain = w["uk"][4 * hd:4 * hd + 4] @ c[j]
            s.append((q[hd, :4] @ k_plain + rot(q[hd, 4:], T - 1) @ rot(down[j, 5:], j)) * 0.3)
        a = torch.softmax(torch.stack(s), 0)
        v = sum(a[j] * (w["uv"][3 * hd:3 * hd + 3] @ c[j]) for j in range(T))
        out.append(v * torch.sigmoid(h[T - 1] @ w["g"][hd]))
    want = torch.cat(out) @ w["o"].T
    assert torch.allclose(got[T - 1], want, rtol=1e-10, atol=1e-12)
