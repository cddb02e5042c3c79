"""Which kernel and which tile a shape gets: pure functions of the shape, checked without a GPU."""


def test_tile_widths_the_tcgen05_product_chooses():
    from hk_b200.csrc import gemm_fast
    cfg = gemm_fast.tc_config
    assert cfg(2048, 24576, 4096, 148, swiglu=True) == (256, 1)         # 1,536 tiles: the widest
    assert cfg(2048, 6144, 4096, 148) == (240, 1)                        # 416 tiles in 3 waves instead of 384 of 256
    assert cfg(2048, 4096, 12288, 148) == (240, 1)                       # 288 tiles in 2 waves
    bn, splits = cfg(64, 24576, 4096, 148, swiglu=True)                  # one wave, every SM a tile
    assert splits == 1 and bn % 32 == 0 and 120 <= -(-24576 // bn) <= 148
    bn, splits = cfg(64, 4096, 12288, 148)
    assert bn in (128, 256) and splits > 1                               # narrow output: K slices
