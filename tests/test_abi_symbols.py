"""The C-ABI library builds, loads without a GPU, and exports every symbol the
header declares; calls that need a device fail with a status, not a crash."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "omoknuni_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ob200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_families():
    names = declared_symbols()
    for must in ("ob200_launch_puct_select", "ob200_launch_vl_revert", "ob200_launch_backup",
                 "ob200_launch_encode_gomoku", "ob200_launch_conv3x3", "ob200_net_infer_gomoku"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in include/omoknuni_b200.h but not exported"


def test_bindings_cover_every_declared_symbol():
    from omoknuni_small_b200 import capi
    missing = [n for n in declared_symbols() if n not in capi.SIGNATURES]
    assert not missing, missing


def test_pure_host_helpers(lib):
    assert lib.ob200_version() == 2
    assert lib.ob200_tree_pitch(225) == 228 and lib.ob200_tree_mask_words(225) == 8
    assert lib.ob200_tree_pitch(4672) == 4672 and lib.ob200_tree_mask_words(4672) == 146
    # 15x15 boards live on a 16x16 grid: 256 positions per board + 2 x 32 guards
    assert lib.ob200_board_tensor_positions(15, 4) == 4 * 256 + 64
    assert lib.ob200_board_tensor_positions(19, 1) == 512 + 64   # 400 rounded up to 128s
    assert lib.ob200_board_tensor_bytes(15, 4, 17) == (4 * 256 + 64) * 24 * 2
    assert lib.ob200_packed_conv3x3_bytes(64, 64) == 9 * 64 * 64 * 2


def test_weight_packing_layout(lib):
    import numpy as np
    from omoknuni_small_b200 import capi
    rng = np.random.default_rng(0)
    w = rng.integers(-8, 8, (64, 17, 3, 3)).astype(np.float32)      # exactly representable in bf16
    scale = np.full(64, 0.5, np.float32)
    packed = capi.pack_conv3x3(w, scale, 64).reshape(9, 64, 8, 8)    # [tap][cout][16-byte chunk][8]
    vals = (packed.astype(np.uint32) << 16).view(np.float32)
    for tap in (0, 4, 8):
        for co in (0, 5, 63):
            row = np.empty(64, np.float32)
            for chunk in range(8):                                    # undo the 128-byte swizzle
                row[chunk * 8:(chunk + 1) * 8] = vals[tap, co, chunk ^ (co % 8)]
            assert np.array_equal(row[:17], w[co, :, tap // 3, tap % 3] * 0.5)
            assert not row[17:].any()                                 # channels >= 17 carry zero weights


def test_weight_packing_f16(lib):
    """The fp16 image has the layout of the bf16 one, values rounded to nearest even and saturated."""
    import numpy as np
    from omoknuni_small_b200 import capi
    rng = np.random.default_rng(1)
    w = rng.normal(0, 1, (64, 64, 3, 3)).astype(np.float32)
    w[0, 0, 0, 0], w[1, 0, 0, 0], w[2, 0, 0, 0] = 1e6, -1e6, 3e-8       # beyond the range on both sides, below the subnormals
    packed = capi.pack_conv3x3(w, None, 64, capi.DTYPE_F16).reshape(9, 64, 8, 8)
    vals = packed.view(np.float16).astype(np.float32)
    want = np.clip(w, -65504.0, 65504.0).astype(np.float16).astype(np.float32)
    for tap in range(9):
        for co in (0, 1, 2, 33, 63):
            row = np.empty(64, np.float32)
            for chunk in range(8):
                row[chunk * 8:(chunk + 1) * 8] = vals[tap, co, chunk ^ (co % 8)]
            assert np.array_equal(row, want[co, :, tap // 3, tap % 3])


@pytest.mark.skipif(os.path.exists("/dev/nvidiactl"), reason="a GPU is present")
def test_no_device_is_an_error_not_a_fallback(lib):
    from omoknuni_small_b200 import capi
    with pytest.raises(capi.Error) as e:
        capi.Net(17, 15, 10, 64, 225)
    assert e.value.code == 2     # OB200_ERR_NO_DEVICE
    assert lib.ob200_device_count() == 0
