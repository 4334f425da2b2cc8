"""The plain implementation against the reference's own model code (tests/golden/*.npz, made by make_golden.py), and
its parts against closed forms."""
import math
import os

import numpy as np
import pytest
import torch

import plain_model
from util import make_model_dir, read_weights

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["tiny_llama", "tiny_qwen2"])
def test_logits_equal_the_reference_models(name, tmp_path):
    g = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    d, cfg, _ = make_model_dir(name, tmp_path)
    got = plain_model.forward(cfg, read_weights(d), g["ids"].tolist()).numpy()
    np.testing.assert_allclose(got, g["logits"], rtol=1e-4, atol=2e-5)
    # the reference's paged engine, greedy, two prompts: the same tokens wherever the top two logits are not a near tie
    w = read_weights(d)
    for prompt, want in ((g["ids"][:11].tolist(), g["engine_ids"][0]), (g["ids"][20:25].tolist(), g["engine_ids"][1])):
        ids = list(prompt)
        for t in want:
            lg = plain_model.forward(cfg, w, ids)[-1].numpy()
            top = np.sort(lg)[-2:]
            if top[1] - top[0] > 1e-3:
                assert int(lg.argmax()) == int(t)
            ids.append(int(t))


def test_rope_bands_of_llama3_scaling():
    inv0 = plain_model.rope_inv_freq(16, 10000.0, None)
    rs = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 32}
    inv = plain_model.rope_inv_freq(16, 10000.0, rs)
    wl = 2 * math.pi / inv0
    assert (wl < 8).any() and (wl > 32).any() and ((wl >= 8) & (wl <= 32)).any(), "all three bands are present"
    np.testing.assert_array_equal(inv[wl < 8], inv0[wl < 8])
    np.testing.assert_allclose(inv[wl > 32], inv0[wl > 32] / 8, rtol=1e-7)
    mid = (wl >= 8) & (wl <= 32)
    assert ((inv[mid] < inv0[mid]) & (inv[mid] > inv0[mid] / 8)).all()
    np.testing.assert_allclose(plain_model.rope_inv_freq(16, 1e4, {"type": "linear", "factor": 4.0}), inv0 / 4, rtol=1e-7)
    cos, sin = plain_model.rope_tables(16, 10000.0, None, 5)
    np.testing.assert_allclose(cos[3].numpy(), np.cos(3 * inv0), rtol=1e-6)


def test_rotation_keeps_lengths_and_relative_angles():
    g = torch.Generator().manual_seed(0)
    cos, sin = plain_model.rope_tables(32, 1e6, None, 50)
    q, k = torch.randn(1, 1, 32, generator=g), torch.randn(1, 1, 32, generator=g)
    def dot(pq, pk):
        return float((plain_model.apply_rope(q, cos[pq:pq + 1], sin[pq:pq + 1]) * plain_model.apply_rope(k, cos[pk:pk + 1], sin[pk:pk + 1])).sum())
    assert abs(dot(10, 7) - dot(43, 40)) < 1e-4 and abs(dot(10, 7) - dot(10, 8)) > 1e-4
    r = plain_model.apply_rope(q, cos[9:10], sin[9:10])
    assert abs(float(r.norm()) - float(q.norm())) < 1e-5


def test_attention_mask_and_window():
    T, hd = 9, 8
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(T, 2, hd, generator=g) for _ in range(3))
    k1, v1 = k[:, :1], v[:, :1]
    full = plain_model.attention(q, k1, v1, 0.5, 0).view(T, 2, hd)
    assert torch.allclose(full[0, 0], v1[0, 0]), "position 0 sees itself only"
    win = plain_model.attention(q, k1, v1, 0.5, 3).view(T, 2, hd)
    assert torch.allclose(win[:3], full[:3]) and not torch.allclose(win[5], full[5])
    s = (q[5, 1] @ k1[3:6, 0].T) * 0.5
    assert torch.allclose(win[5, 1], torch.softmax(s, 0) @ v1[3:6, 0], atol=1e-6), "window 3 at position 5: keys 3, 4, 5"


def test_rmsnorm_and_silu():
    x = torch.tensor([[3.0, 4.0]])
    assert torch.allclose(plain_model.rmsnorm(x, torch.tensor([1.0, 2.0]), 0.0), torch.tensor([[3 / math.sqrt(12.5), 8 / math.sqrt(12.5)]]))
    assert torch.allclose(plain_model.silu(torch.tensor([0.0, 2.0])), torch.tensor([0.0, 2.0 / (1 + math.exp(-2.0))]))


def test_sampling_rules():
    lg = np.array([1.0, 3.0, 3.0, -2.0, 0.5], np.float32)
    assert plain_model.sample(lg, [], 0.0, 0, 1.0, 1.0, np.random.default_rng(0)) == 1, "greedy: first index of the maximum"
    assert plain_model.sample(lg, [1, 2], 0.0, 0, 1.0, 4.0, np.random.default_rng(0)) == 0, "penalty divides positive logits"
    pen = plain_model.apply_repetition_penalty(lg, [3], 2.0)
    assert pen[3] == -4.0
    assert np.isinf(plain_model.top_k_filter(lg.astype(np.float64), 1)).sum() == 3, "ties at the k-th value stay"
    kept = np.isfinite(plain_model.top_p_filter(lg.astype(np.float64), 0.5))
    assert kept.tolist() == [False, True, True, False, False]
    assert np.isfinite(plain_model.top_p_filter(lg.astype(np.float64), 1e-9)).sum() == 1, "the top one always stays"
    draws = [plain_model.sample(lg, [], 1.0, 0, 1.0, 1.0, np.random.default_rng(s)) for s in range(300)]
    p = plain_model.softmax64(lg)
    assert abs(draws.count(1) / 300 - p[1]) < 0.1 and draws.count(3) < 10
    a = [plain_model.sample(lg, [], 0.8, 3, 0.9, 1.1, np.random.default_rng(5)) for _ in range(1)]
    b = [plain_model.sample(lg, [], 0.8, 3, 0.9, 1.1, np.random.default_rng(5)) for _ in range(1)]
    assert a == b


def test_two_restatements_of_the_filters_agree():
    """The product's host sampler (used for rows with a repetition penalty) and the plain kernel table's filtered
    sampling (the reference of the device kernel) are written apart from each other; on rows with many equal values,
    masked tokens and every mix of top-k and top-p they must pick the same token from the same uniform number."""
    import torch
    from plain_ops import PlainOps
    from fusezap_core_b200.sampling import RequestSampler
    from fusezap_core_b200 import SamplingParams
    rng = np.random.default_rng(3)
    V = 257
    for trial in range(40):
        lg = (rng.standard_normal(V) * 3).astype(np.float32)
        if trial % 3 == 0:
            lg = np.round(lg * 2) / 2
        if trial % 5 == 0:
            lg[::4] = -np.inf
        k = [0, 2, 7, 50, V, V + 3][trial % 6]
        p = [1.0, 0.95, 0.5, 0.1][(trial // 2) % 4]
        t = [0.8, 1.7][trial % 2]
        seed = 100 + trial
        sampler = RequestSampler(SamplingParams(temperature=float(np.float32(t)), top_k=k, top_p=float(np.float32(p)), seed=seed))
        want = sampler.host_choice(lg, [])
        u = np.random.default_rng(seed).random()
        out = torch.empty(1, dtype=torch.int32)
        PlainOps().sample_filtered(torch.from_numpy(lg)[None], torch.tensor([t], dtype=torch.float32),
                                   torch.tensor([k], dtype=torch.int32), torch.tensor([p], dtype=torch.float32),
                                   torch.tensor([u], dtype=torch.float64), out)
        assert int(out[0]) == want, (trial, k, p, t)
