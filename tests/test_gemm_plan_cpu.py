"""The GEMM launcher's tile / split-K planner, exercised through the native library without a GPU.

The reference picks its GEMM variant by shape thresholds (FINAL_CLEAN_CODE_/src/kernels/gemm.cu:1784-1998: atomic
split-K for tall-skinny weight gradients, tile-size dispatch by M and N); the plan here comes from a cost model over
tile shapes, CTA pairs and K splits, and these cases pin its decisions on the shapes the models produce."""
import ctypes

import pytest

from cme213_final_project_b200 import ops


def _plan(M, N, K, batch=1, plain=True, ws=1 << 30, sms=148, pairs=74, force_bn=0, force_splits=0):
    lib = ops.host_lib()
    if lib is None:
        pytest.skip("native library not built")
    out = (ctypes.c_int * 3)()
    rc = lib.cme_gemm_plan(M, N, K, batch, int(plain), ctypes.c_longlong(ws), sms, pairs, force_bn, force_splits, out)
    assert rc == 0
    return {"bn": out[0], "pair": bool(out[1]), "splits": out[2]}


def test_large_products_use_cta_pairs_without_splitting():
    for shape in [(16384, 3072, 768), (16384, 2304, 768), (16384, 768, 3072), (16384, 50304, 768), (8192, 8192, 8192)]:
        p = _plan(*shape)
        assert p == {"bn": 256, "pair": True, "splits": 1}, (shape, p)


def test_weight_gradients_split_k_to_fill_the_machine():
    # 768 x 3072 is 36 pair tiles for 74 pairs: two splits; 768 x 768 is 9 tiles: eight
    assert _plan(768, 3072, 16384) == {"bn": 256, "pair": True, "splits": 2}
    assert _plan(3072, 768, 16384) == {"bn": 256, "pair": True, "splits": 2}
    assert _plan(768, 768, 16384)["splits"] == 8
    # 192 pair tiles over 74 pairs leave a 0.6 wave: three splits even it out when the workspace allows
    assert _plan(16384, 768, 50304)["splits"] == 3
    assert _plan(16384, 768, 50304, ws=64 << 20)["splits"] == 1


def test_split_k_needs_plain_epilogue_workspace_and_enough_depth():
    assert _plan(768, 3072, 16384, plain=False)["splits"] == 1
    assert _plan(768, 3072, 16384, ws=0)["splits"] == 1
    assert _plan(768, 768, 256)["splits"] == 1            # four k-blocks in all: nothing to split


def test_small_and_narrow_products_use_narrow_single_cta_tiles():
    assert _plan(2048, 65, 256) == {"bn": 64, "pair": False, "splits": 1}
    assert _plan(128, 128, 128)["pair"] is False          # one row block: nothing for a second CTA
    assert _plan(2048, 512, 128)["bn"] in (64, 128)


def test_no_cluster_launches_falls_back_to_single_cta_tiles():
    p = _plan(16384, 3072, 768, pairs=0)
    assert p["pair"] is False and p["bn"] == 256


def test_forced_choices_are_respected():
    assert _plan(16384, 3072, 768, force_bn=128)["bn"] == 128
    assert _plan(16384, 3072, 768, force_bn=512) == {"bn": 256, "pair": True, "splits": 1}
    assert _plan(768, 3072, 16384, force_splits=4)["splits"] == 4
