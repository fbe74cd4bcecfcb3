"""The host-side choices of tile shapes and splits: pure functions of the sizes, checked on the CPU."""
import itertools

from llm_inference_lab_b200.kernels import ops


def test_decode_splits_fit_the_gpu_and_the_cluster():
    """Splits never ask for more CTAs than the SMs hold at once, never leave a CTA without keys,
    and the cluster path (2..8 splits) is only taken while all CTAs are resident together."""
    for n_decode, n_kv, group, kv, (keys, per_sm) in itertools.product(
            (1, 2, 8, 32, 64, 200), (1, 2, 4, 8), (1, 7, 16, 20), (1, 100, 640, 2048, 4096, 32768),
            ((128, 2), (192, 1))):
        s = ops.decode_splits(n_decode, n_kv, group, kv, keys, per_sm)
        ctas = n_decode * n_kv * (-(-group // 16))
        assert 1 <= s <= 32
        if s > 1:
            assert (s - 1) * keys < kv, "a split without keys"
            assert ctas * s <= per_sm * ops.sm_count(), "a second round of CTAs"


def test_decode_splits_short_contexts_are_not_split():
    assert ops.decode_splits(8, 2, 7, 100) == 1
    assert ops.decode_splits(1, 1, 1, 1) == 1


def test_decode_splits_benchmark_shapes():
    # batch 8 of the 0.5B shape at 640 keys: one round of the warps per CTA, merged in the cluster
    assert ops.decode_splits(8, 2, 7, 640) == 5
    # heads of 128 (12 warps x 16 keys per round, one CTA per SM), 32 requests: no room to split
    assert ops.decode_splits(32, 4, 7, 4096, 192, 1) == 1


def test_prefill_tiles_cover_the_cases_they_were_measured_on():
    pick = ops._pick_prefill_tiles
    # down projection of the 0.5B shape: one wave of 128-wide tiles, K split to fill it
    assert pick(2048, 896, 4864, True) == ("tc", 128, 1)
    assert pick(1024, 896, 4864, True) == ("tc", 128, 2)
    assert pick(512, 896, 4864, True) == ("tc", 128, 4)
    # the same product may not be split when its consumer cannot sum partial products
    assert pick(512, 896, 4864, False) == ("tc", 128, 1)
    # short K is never split
    assert pick(512, 896, 896, True) == ("tc", 128, 1)
    # long K and enough tiles for most pairs of SMs: the pair kernel
    assert pick(4096, 896, 4864, True)[0] == "pair"
    assert pick(2048, 3584, 18944, True)[0] == "pair"
    # beyond one wave the width with the cheaper waves
    assert pick(1024, 3584, 1536, True) == ("tc", 256, 1)


def test_prefill_tiles_are_always_a_shape_the_kernels_take():
    for T, n_out, K, partial in itertools.product((129, 256, 1000, 2048, 8192, 50000), (8, 896, 1152, 9728, 151936),
                                                  (64, 896, 4864, 18944), (False, True)):
        kind, bn, splits = ops._pick_prefill_tiles(T, n_out, K, partial)
        assert kind in ("tc", "pair") and bn in (128, 256) and splits >= 1
        if not partial or kind == "pair":
            assert splits == 1
        if splits > 1:
            assert -(-K // 64) // splits >= 16, "a split with too few k-tiles"
            assert -(-T // 128) * -(-n_out // bn) * splits <= ops.sm_count()
