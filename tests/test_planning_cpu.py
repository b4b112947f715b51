"""Host-side planning logic that needs no GPU: segment planning, slice widths, shard bounds."""
import pytest


def test_plan_segments():
    from palimpsa_b200.ops.palimpsa._core import plan_segments, segment_len
    assert plan_segments(8, 4096, 6, 128, 128) == 1        # 384 (sequence, head, tile) CTAs fill the GPU
    assert plan_segments(4, 4096, 6, 128, 128) == 1        # 192 CTAs: still above the SM count
    assert plan_segments(3, 4096, 6, 128, 128) == 16       # 144 CTAs: 256-token segments
    assert plan_segments(1, 131072, 12, 128, 128) == 32    # long sequence: capped at 32 pieces
    assert plan_segments(1, 1024, 2, 64, 64) == 1          # short sequences never
    assert plan_segments(1, 2048, 1, 64, 64) == 8
    # with a backward to follow, the backward grid decides (one CTA of up to 12 warps per SM, 148 SMs assumed here)
    kw = dict(backward=True)
    assert plan_segments(8, 4096, 6, 128, 128, **kw) == 1     # 288 CTAs of 22 rows = 1.95 waves
    assert plan_segments(4, 4096, 6, 128, 128, **kw) == 1     # 144 CTAs = 0.97 of a wave
    assert plan_segments(5, 4096, 6, 128, 128, **kw) == 16    # 180 CTAs = 1.2 waves: the second one mostly idle
    assert plan_segments(2, 4096, 6, 128, 128, **kw) == 16    # 72 CTAs: half the SMs idle
    assert plan_segments(8, 4096, 16, 48, 48, **kw) == 1      # the 170M model's heads: 128 CTAs = 0.86 of a wave
    assert plan_segments(8, 4096, 12, 64, 64, **kw) == 16     # 192 CTAs = 1.3 waves
    assert plan_segments(8, 1024, 12, 64, 64, **kw) == 1      # short sequences never
    # packed rows: only the document count is known; segments when the documents alone cannot fill one wave
    assert plan_segments(7, 16384, 16, 48, 48, packed=True, **kw) == 32     # 112 CTAs: the longest document binds
    assert plan_segments(14, 32768, 16, 48, 48, packed=True, **kw) == 1     # 224 CTAs, started longest first
    assert plan_segments(14, 32768, 6, 128, 128, packed=True, **kw) == 1
    assert plan_segments(3, 32768, 6, 128, 128, packed=True) == 32          # forward only: 144 forward CTAs
    for T, G in ((4096, 16), (333, 3), (17, 4), (1, 1)):
        L = segment_len(T, G)
        assert L % 16 == 0 and L * G >= T and L >= 16


def test_ramped_widths():
    from palimpsa_b200.host_pipeline import ramped_widths
    assert ramped_widths(8) == [1, 2, 2, 2, 1]
    assert ramped_widths(9, middle=3) == [1, 3, 3, 1, 1]
    assert ramped_widths(1) == [1] and ramped_widths(2) == [1, 1]
    for b in range(1, 40):
        w = ramped_widths(b)
        assert sum(w) == b and min(w) >= 1 and w[0] == 1 and w[-1] == 1


def test_shard_bounds_cover_without_overlap():
    from palimpsa_b200.parallel import shard_bounds
    for n in (0, 1, 7, 8, 131072):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def test_layer_wrappers_reject_cpu_tensors():
    import torch
    from palimpsa_b200.layers import layer_epilogue, layer_prologue
    x = torch.zeros(1, 2, 2, 8)
    with pytest.raises(RuntimeError):
        layer_epilogue(x, None, None, torch.ones(8))
    with pytest.raises(RuntimeError):
        layer_prologue(x, x, x, x, torch.zeros(1, 2, 2), torch.zeros(1, 2, 2), torch.zeros(2), torch.zeros(2))


def test_missing_library_is_a_loud_error(monkeypatch, tmp_path):
    """No CPU or PyTorch fallback: without the built CUDA library every entry fails with a clear message."""
    from palimpsa_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libpalimpsa_b200.so"))
    with pytest.raises(_lib.PalimpsaLibraryError, match="no CPU or PyTorch fallback"):
        _lib.lib()


def test_forward_tile_rows_from_the_library():
    """Pure host function of the C ABI: rows of one forward CTA per head shape (what plan_segments counts CTAs with)."""
    from palimpsa_b200 import _lib
    lib = _lib.lib()
    assert lib.palimpsa_fwd_tile_rows(128, 128) == 16
    assert lib.palimpsa_fwd_tile_rows(64, 64) == 32
    assert lib.palimpsa_fwd_tile_rows(64, 8) == 16         # short d_v: one warp instead of two, half the tile
    assert lib.palimpsa_fwd_tile_rows(300, 64) == 0        # d_k above the supported maximum
    assert lib.palimpsa_fwd_tile_rows(48, 48) == 48        # three warps: no idle rows at the 170M model's heads
    assert lib.palimpsa_bwd_tile_rows(128, 128, _lib.BF16, 0) == 22   # 11 warps x 2 rows: 6 tiles = 132 rows
    assert lib.palimpsa_bwd_tile_rows(48, 48, _lib.BF16, 0) == 48     # 6 warps x 8 rows
    assert lib.palimpsa_bwd_tile_rows(48, 96, _lib.BF16, 0) == 48
    assert lib.palimpsa_bwd_tile_rows(64, 64, _lib.BF16, 0) == 32
    assert lib.palimpsa_bwd_tile_rows(300, 64, _lib.BF16, 0) == 0
    assert lib.palimpsa_bwd_tile_rows(64, 64, 99, 0) == 0             # unknown element type
    assert lib.palimpsa_last_error_string(_lib.E_SYMBOL).startswith(b"the library's own scratch array")
