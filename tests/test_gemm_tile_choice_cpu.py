"""The fp32 GEMM engine's choice between 128 x 128 and 128 x 256 output tiles is host arithmetic
(waves of tiles over the SMs, a wide tile counted as 1.6 narrow ones), so it is checked without a
GPU: the shapes of the benchmark's products and the properties the driver relies on."""

from onecompression_b200 import _lib

SMS = 148
SKIP_UPPER = 1          # OC_GEMM_SKIP_UPPER_TILES
NARROW, WIDE = 1, 2


def choice(m, n, batch=1, flags=0, sms=SMS):
    return _lib.load().oc_gemm_tile_choice(m, n, batch, flags, sms)


def waves(tiles, sms=SMS):
    return -(-tiles // sms)


def test_products_of_the_benchmark():
    # dense QEP products W·C: enough tiles to fill the SMs several times -> wide
    assert choice(4096, 4096) == WIDE
    assert choice(28672, 4096) == WIDE
    assert choice(4096, 14336) == WIDE
    # near trailing update (<= 384 columns) and small products: one wave either way -> narrow
    assert choice(4096, 384) == NARROW
    assert choice(4096, 128) == NARROW
    assert choice(1024, 1024) == NARROW
    # far trailing update of a 4096-row layer, 3584 columns
    assert choice(4096, 3584) == WIDE
    # Cholesky outer update (lower tiles only): d = 14336 pays, d = 4096 does not
    assert choice(13824, 13824, flags=SKIP_UPPER) == WIDE
    assert choice(3584, 3584, flags=SKIP_UPPER) == NARROW


def test_rule_is_waves_times_cost():
    for m, n, batch in ((4096, 4096, 1), (300, 200, 1), (2880, 2880, 32), (128, 256, 1), (777, 5000, 3),
                        (14336, 640, 1), (64, 136, 1)):
        tm = -(-m // 128)
        narrow = waves(batch * tm * -(-n // 128))
        wide = 1.6 * waves(batch * tm * -(-n // 256))
        assert choice(m, n, batch) == (WIDE if wide < narrow else NARROW), (m, n, batch)


def test_degenerate_and_forced():
    lib = _lib.load()
    assert choice(0, 128) == NARROW and choice(128, 0) == NARROW and choice(128, 128, sms=0) == NARROW
    old = lib.oc_set_gemm_tile_shape(1)
    try:
        assert choice(4096, 4096) == NARROW
        lib.oc_set_gemm_tile_shape(2)
        assert choice(128, 128) == WIDE
    finally:
        lib.oc_set_gemm_tile_shape(old)
    assert choice(4096, 4096) == WIDE
