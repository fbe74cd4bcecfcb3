"""The plain implementation itself: properties each part must have, whatever the weights (no GPU)."""
import numpy as np
import pytest

from helpers import TINY_A, TINY_C, make_model_folder
from plain_qwen2 import (plain_attention, plain_forward, plain_greedy, plain_inv_freq, plain_linear, plain_rms_norm,
                         plain_rope, plain_sample, plain_silu, plain_uniform, read_model_folder)


def test_rms_norm_is_scale_free_and_uses_the_true_width():
    rng = np.random.default_rng(0)
    x, w = rng.standard_normal((3, 10)), rng.standard_normal(10)
    y = plain_rms_norm(x, w, 0.0)
    assert np.allclose(plain_rms_norm(7.0 * x, w, 0.0), y)
    assert np.allclose((y / w) ** 2 @ np.ones(10) / 10, 1.0)
    assert np.allclose(plain_rms_norm(np.zeros((1, 4)), np.ones(4), 1e-6), 0.0)


def test_rope_is_a_rotation_that_depends_on_relative_position():
    rng = np.random.default_rng(1)
    q, k = rng.standard_normal((1, 1, 32)), rng.standard_normal((1, 1, 32))
    assert np.allclose(plain_rope(q, [0], 1e4), q), "position 0 leaves a head as it is"
    assert np.allclose(np.linalg.norm(plain_rope(q, [77], 1e4)), np.linalg.norm(q))
    dots = [float(plain_rope(q, [m], 1e4).ravel() @ plain_rope(k, [m - 5], 1e4).ravel()) for m in (5, 60, 999)]
    assert np.allclose(dots, dots[0], atol=1e-3), "q_m . k_n depends on m - n only"
    inv = plain_inv_freq(32, 1e4)
    assert inv.dtype == np.float32 and inv[0] == 1.0 and np.isclose(inv[-1], 1e4 ** (-30 / 32))
    # split-half pairing: element i turns with element i + d/2
    e = np.zeros((1, 1, 8)); e[0, 0, 1] = 1.0
    out = plain_rope(e, [3], 100.0)[0, 0]
    assert np.count_nonzero(np.abs(out) > 1e-12) == 2 and abs(out[1]) > 0 and abs(out[5]) > 0


def test_attention_is_causal_grouped_and_windowed():
    rng = np.random.default_rng(2)
    T, n_h, n_kv, d = 9, 4, 2, 8
    q, k, v = rng.standard_normal((T, n_h, d)), rng.standard_normal((T, n_kv, d)), rng.standard_normal((T, n_kv, d))
    pos = np.arange(T)
    out = plain_attention(q, k, v, pos)
    assert np.allclose(out[0], v[0][[0, 0, 1, 1]]), "the first row sees one key; heads 0,1 use kv head 0"
    k2, v2 = k.copy(), v.copy()
    k2[5:], v2[5:] = 9.0, -9.0
    assert np.allclose(plain_attention(q, k2, v2, pos)[:5], out[:5]), "later keys do not matter"
    # brute force for one element
    s = (k[:7, 1] @ q[6, 3]) / np.sqrt(d)
    w = np.exp(s - s.max()); w /= w.sum()
    assert np.allclose(out[6, 3], w @ v[:7, 1])
    win = plain_attention(q, k, v, pos, window=3)
    assert np.allclose(win[:3], out[:3]) and not np.allclose(win[3:], out[3:])
    s = (k[4:7, 0] @ q[6, 0]) / np.sqrt(d)
    w = np.exp(s - s.max()); w /= w.sum()
    assert np.allclose(win[6, 0], w @ v[4:7, 0]), "window 3 at position 6 sees keys 4, 5, 6"


def test_linear_silu_and_sampling_rules():
    assert np.allclose(plain_linear([[1, 2]], [[3, 4], [5, 6]], [1, 1]), [[12, 18]])
    assert np.allclose(plain_silu([0.0, 1.0]), [0.0, 1 / (1 + np.exp(-1))])
    assert plain_sample([1.0, 3.0, 3.0, 2.0], 0, 0, 0)[0] == 1, "ties go to the smallest index"
    u = plain_uniform(7, 5, 1000)
    assert ((u > 0) & (u < 1)).all() and abs(u.mean() - 0.5) < 0.05
    assert not np.allclose(u, plain_uniform(8, 5, 1000)) and not np.allclose(u, plain_uniform(7, 6, 1000))
    assert np.allclose(u[:10], plain_uniform(7, 5, 10)), "a draw depends on (seed, position, index) only"
    picks = [plain_sample(np.log([0.7, 0.2, 0.1]), 1.0, s, 0)[0] for s in range(2000)]
    freq = np.bincount(picks, minlength=3) / 2000
    assert np.allclose(freq, [0.7, 0.2, 0.1], atol=0.04), "Gumbel-max samples from softmax(logits / T)"


@pytest.mark.parametrize("raw", [TINY_A, TINY_C])
def test_forward_is_causal_and_reads_the_folder(tmp_path, raw):
    folder = make_model_folder(str(tmp_path), raw, seed=4, dtype="float32")
    cfg, w = read_model_folder(folder)
    ids = list(np.random.default_rng(3).integers(0, raw["vocab_size"], 40))
    full = plain_forward(cfg, w, ids)
    assert full.shape == (40, raw["vocab_size"]) and np.isfinite(full).all()
    assert np.allclose(plain_forward(cfg, w, ids[:23]), full[:23], atol=1e-9), "a prefix gives the same logits"
    other = ids[:30] + [(t + 1) % raw["vocab_size"] for t in ids[30:]]
    assert np.allclose(plain_forward(cfg, w, other)[:30], full[:30], atol=1e-9)
    if raw.get("use_sliding_window"):
        no_window = dict(cfg, use_sliding_window=False)
        far = plain_forward(no_window, w, ids)
        assert np.allclose(far[:20], full[:20], atol=1e-9), "within the window nothing changes"
        assert not np.allclose(far[25:], full[25:], atol=1e-6), "beyond it the windowed layers see less"
    out = plain_greedy(cfg, w, ids[:5], 3)
    assert len(out) == 3 and out[0] == int(np.argmax(plain_forward(cfg, w, ids[:5])[-1]))


def test_twins_of_an_engines_precision(tmp_path):
    """The plain functions as twins: bfloat16 rounding is round-to-nearest-even (checked against the
    tensor library's cast, specials included); inside `plain_precision` the parts compute in 32-bit or
    round every operator's result, outside they are the 64-bit yardstick again; the twins lie near the
    yardstick by their precision's size, the bfloat16 one farther than the 32-bit one."""
    import torch

    import plain_qwen2 as pq
    from plain_qwen2 import plain_precision, read_model_folder, round_bfloat16

    x = (np.random.default_rng(0).standard_normal(50000) * 3.7).astype(np.float32)
    x[:6] = [0.0, np.inf, -np.inf, 1e-40, 3.3895314e38, -1.0000001]
    assert np.array_equal(round_bfloat16(x), torch.from_numpy(x).to(torch.bfloat16).float().numpy())

    folder = make_model_folder(str(tmp_path / "m"), TINY_A, 0, "float32")
    cfg, w = read_model_folder(folder)
    ids = [int(t) for t in np.random.default_rng(1).integers(0, TINY_A["vocab_size"], 40)]
    ref = plain_forward(cfg, w, ids)
    with plain_precision(np.float32):
        f32 = plain_forward(cfg, w, ids)
        assert f32.dtype == np.float32
    with plain_precision(edge=round_bfloat16):
        b16 = plain_forward(cfg, w, ids)
    assert pq._COMPUTE is np.float64 and pq._EDGE is None, "the yardstick is back"
    assert np.array_equal(plain_forward(cfg, w, ids), ref)
    scale = np.abs(ref).max()
    e32, e16 = np.abs(f32 - ref).max() / scale, np.abs(b16 - ref).max() / scale
    assert 0 < e32 < 1e-5 and 1e-4 < e16 < 0.05
