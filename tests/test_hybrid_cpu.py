"""Hybrid operator registration: schemas, fake (meta) shapes, knobs, loader idempotence (CPU)."""
import pytest
import torch

from sparser_faster_llms_b200 import dropin, sparse_ops
from sparser_faster_llms_b200.sparse_ops_loader import load_sparse_ops


@pytest.fixture(scope="module", autouse=True)
def ops():
    load_sparse_ops()
    load_sparse_ops()


def test_operator_schemas_match_the_reference_names_and_order():
    fwd = torch.ops.sparse_ops.ff_forward_gated.default._schema
    assert [a.name for a in fwd.arguments] == ["X", "G", "K", "V"]
    assert len(fwd.returns) == 6
    bwd = torch.ops.sparse_ops.ff_backward_gated.default._schema
    assert [a.name for a in bwd.arguments] == ["X", "G", "K", "V", "P", "R", "T", "gR", "gl0", "gl1"]
    assert len(bwd.returns) == 4
    raw = torch.ops.sparse_ops.ell_spmm_raw.default._schema
    assert [a.name for a in raw.arguments] == ["ell_vals", "ell_cols", "row_counts", "B", "M", "K",
                                               "N", "ell_stride", "overflow_threshold"]
    for name in ("set_ell_width_regular", "set_ell_width_transpose", "set_tail_rows_regular",
                 "set_tail_rows_transpose", "set_discard_overflow",
                 "get_last_transpose_overflow_count"):
        assert hasattr(torch.ops.sparse_ops_config, name)
    assert hasattr(torch.ops.sparse_ops_perf, "print_report")
    assert hasattr(torch.ops.sparse_ops_perf, "reset_stats")


def test_fake_tensors_give_shapes_without_a_gpu():
    x = torch.empty(2, 8, 512, dtype=torch.bfloat16, device="meta")
    w = torch.empty(1024, 512, dtype=torch.bfloat16, device="meta")
    out, l0, l1, P, R, T = torch.ops.sparse_ops.ff_forward_gated(x, w, w, w)
    assert out.shape == x.shape and l0.shape == () and l1.shape == ()
    assert P.shape == (16, 4 * 64) and P.dtype == torch.int32
    dx, dg, dk, dv = torch.ops.sparse_ops.ff_backward_gated(x, w, w, w, P, R, T, out, l0, l1)
    assert dx.shape == x.shape and dg.shape == dk.shape == dv.shape == w.shape


def test_knobs_map_ell_width_to_slab_width():
    try:
        for width, cf in ((64, 8), (124, 8), (128, 4), (252, 4), (256, 2), (1024, 2)):
            torch.ops.sparse_ops_config.set_ell_width_regular(width)
            assert sparse_ops.compression_factor() == cf
        with pytest.raises(Exception):
            torch.ops.sparse_ops_config.set_tail_rows_regular(-1)
    finally:
        torch.ops.sparse_ops_config.set_ell_width_regular(128)
    with pytest.raises(RuntimeError, match="No backward pass"):
        if sparse_ops._LAST_TRANSPOSE_OVERFLOW is None:
            torch.ops.sparse_ops_config.get_last_transpose_overflow_count()
        else:
            raise RuntimeError("No backward pass")


def test_cpu_tensors_are_rejected():
    x = torch.zeros(1, 4, 256, dtype=torch.bfloat16)
    w = torch.zeros(512, 256, dtype=torch.bfloat16)
    with pytest.raises(Exception):
        torch.ops.sparse_ops.ff_forward_gated(x, w, w, w)


def test_dropin_registers_the_loader_name():
    import sys
    dropin.install(twell=False)
    from sparser_faster_llms_b200 import sparse_ops_loader
    assert sys.modules[dropin.LOADER_NAME] is sparse_ops_loader
    dropin.uninstall()
