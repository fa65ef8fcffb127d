"""The byte counts that bench.py's roofline fractions rest on, against the figures worked out by
hand for the three published shapes: every matrix of the model once, and the keys and values of
the live requests."""
import bench


def test_bytes_a_decode_step_has_to_read():
    tiny = bench.SHAPES["tinyllama"]["config"]
    per_layer, weights, cache = bench.model_bytes_and_flops(tiny, 22, 8, 2048)
    assert per_layer == 44_040_192                        # parameters of one layer's five matrices
    assert weights == 2_068_840_448                       # 22 layers and the head, bfloat16
    assert cache == 8 * 2048 * 22_528                     # 22 layers x 2 x 256 channels x 2 bytes a position
    l2 = bench.SHAPES["llama2-7b"]["config"]
    _, weights, cache = bench.model_bytes_and_flops(l2, 32, 1, 4096)
    assert weights == 13_214_154_752 and cache == 4096 * 524_288
    l3 = bench.SHAPES["llama3-8b"]["config"]
    _, weights, cache = bench.model_bytes_and_flops(l3, 32, 64, 8192)
    assert weights == 15_009_316_864 and cache == 64 * 8192 * 131_072
    # fewer layers than the shape has: the layers' share shrinks, the head's does not
    _, fewer, _ = bench.model_bytes_and_flops(l3, 8, 1, 0)
    head = 128_256 * 4096 * 2
    assert (weights - head) == 4 * (fewer - head)


def test_shapes_are_the_published_ones_and_the_peaks_have_a_source():
    assert bench.PREFILL_TOKENS == 2048
    assert [bench.SHAPES[k]["context"] for k in ("tinyllama", "llama2-7b", "llama3-8b")] == [2048, 4096, 8192]
    hbm, tflops, source = bench.peaks()
    assert source in ("measured", "fallback") and 1000 < hbm < 10000 and 100 < tflops < 5000
    if source == "fallback":
        assert (hbm, tflops) == (6650.0, 1590.0)
