"""Packing tensors into per-dtype buffers and back, NaN scans and difference
reports, case by case (the reference pins these in `awex/tests/test_tensor_utils.py`
and `awex/tests/test_weights_util.py`)."""

import io
from contextlib import redirect_stdout

import pytest
import torch

from awex_b200.utils.tensor_util import (
    check_and_log_nan_values, compare_and_log_tensor_differences, group_tensors_by_shape_and_dtype, reconstruct_tensors_from_groups,
)


def logged(fn, *args, **kwargs):
    out = io.StringIO()
    with redirect_stdout(out):
        result = fn(*args, **kwargs)
    return result, out.getvalue()


# ---- grouping ----------------------------------------------------------------------------------------
def test_grouping_nothing_gives_nothing():
    assert group_tensors_by_shape_and_dtype([]) == ([], [])
    assert reconstruct_tensors_from_groups([], []) == []


def test_one_tensor_becomes_one_flat_buffer():
    t = torch.randn(3, 4)
    groups, meta = group_tensors_by_shape_and_dtype([t])
    assert len(groups) == 1 and groups[0].shape == (12,) and torch.equal(groups[0], t.reshape(-1))
    assert meta == [{"original_index": 0, "group_index": 0, "offset": 0, "size": 12, "shape": (3, 4), "dtype": torch.float32}]


def test_equal_and_different_shapes_of_one_dtype_share_a_buffer():
    tensors = [torch.randn(2, 3), torch.randn(2, 3), torch.randn(4), torch.randn(1, 5, 2)]
    groups, meta = group_tensors_by_shape_and_dtype(tensors)
    assert len(groups) == 1 and groups[0].numel() == 6 + 6 + 4 + 10
    assert [m["offset"] for m in meta] == [0, 6, 12, 16] and [m["shape"] for m in meta] == [(2, 3), (2, 3), (4,), (1, 5, 2)]


def test_each_dtype_gets_its_own_buffer():
    tensors = [torch.randn(4), torch.arange(6, dtype=torch.int64), torch.randn(3).to(torch.bfloat16), torch.randn(2, 2)]
    groups, meta = group_tensors_by_shape_and_dtype(tensors)
    assert sorted(str(g.dtype) for g in groups) == ["torch.bfloat16", "torch.float32", "torch.int64"]
    by_index = {m["original_index"]: m for m in meta}
    assert by_index[0]["group_index"] == by_index[3]["group_index"] != by_index[1]["group_index"]


def test_a_byte_limit_splits_buffers_and_an_oversize_tensor_travels_alone():
    tensors = [torch.ones(4), torch.ones(4), torch.ones(4), torch.ones(100)]
    groups, meta = group_tensors_by_shape_and_dtype(tensors, max_tensor_size=32)  # two 16-byte tensors per buffer
    assert [g.numel() for g in groups] == [8, 4, 100]
    back = reconstruct_tensors_from_groups(groups, meta)
    assert all(torch.equal(a, b) for a, b in zip(tensors, back))


def test_scalars_and_high_rank_tensors_survive():
    tensors = [torch.tensor(3.5), torch.randn(2, 3, 4, 5), torch.randn(1, 1, 7)]
    groups, meta = group_tensors_by_shape_and_dtype(tensors)
    back = reconstruct_tensors_from_groups(groups, meta)
    assert [tuple(b.shape) for b in back] == [(), (2, 3, 4, 5), (1, 1, 7)]
    assert all(torch.equal(a, b) for a, b in zip(tensors, back))


def test_only_dense_tensors_are_accepted():
    with pytest.raises(ValueError):
        group_tensors_by_shape_and_dtype([torch.ones(2).to_sparse()])
    with pytest.raises(ValueError):
        group_tensors_by_shape_and_dtype(["not a tensor"])


# ---- reconstruction -------------------------------------------------------------------------------
def test_reconstruction_gives_views_in_the_original_order():
    tensors = [torch.randn(2, 2), torch.arange(5), torch.randn(3), torch.arange(4).reshape(2, 2)]
    groups, meta = group_tensors_by_shape_and_dtype(tensors)
    shuffled = list(reversed(meta))  # the order of the metadata does not matter
    back = reconstruct_tensors_from_groups(groups, shuffled)
    assert all(torch.equal(a, b) for a, b in zip(tensors, back))
    back[0].zero_()
    first = next(m for m in meta if m["original_index"] == 0)
    assert not groups[first["group_index"]][first["offset"]: first["offset"] + 4].any()  # a view: writes land in the buffer


def test_reconstruction_refuses_metadata_that_does_not_fit_the_buffers():
    tensors = [torch.randn(4), torch.arange(3)]
    groups, meta = group_tensors_by_shape_and_dtype(tensors)
    with pytest.raises(ValueError, match="group"):
        reconstruct_tensors_from_groups(groups[:1], meta)  # a group is missing
    with pytest.raises(ValueError, match="group"):
        reconstruct_tensors_from_groups([], meta)
    with pytest.raises(ValueError, match="exceeds"):
        reconstruct_tensors_from_groups([g[:1] for g in groups], meta)  # buffers shorter than the metadata says
    with pytest.raises(ValueError, match="every original index"):
        reconstruct_tensors_from_groups(groups, [m for m in meta if m["original_index"] != 0])
    with pytest.raises((ValueError, TypeError, AttributeError)):
        reconstruct_tensors_from_groups([None, None], meta)


@pytest.mark.parametrize("dtypes", [(torch.float32,), (torch.float16, torch.bfloat16), (torch.float32, torch.int32, torch.uint8, torch.bool)])
def test_round_trip_of_many_tensors(dtypes):
    torch.manual_seed(0)
    tensors = []
    for i in range(40):
        shape = tuple(int(x) for x in torch.randint(1, 6, (int(torch.randint(1, 4, ())),)))
        tensors.append((torch.randn(shape) * 10).to(dtypes[i % len(dtypes)]))
    groups, meta = group_tensors_by_shape_and_dtype(tensors, max_tensor_size=256)
    assert len(groups) >= len(dtypes)
    back = reconstruct_tensors_from_groups(groups, meta)
    assert all(a.dtype == b.dtype and torch.equal(a, b) for a, b in zip(tensors, back))


# ---- NaN scan --------------------------------------------------------------------------------------
def test_clean_tensors_report_nothing():
    for t in (torch.ones(3, 3), torch.empty(0), torch.ones(3, dtype=torch.int32), torch.tensor([float("inf"), -float("inf"), 1.0])):
        found, text = logged(check_and_log_nan_values, t, "t")
        assert not found and text == ""  # infinities are not NaNs


def test_nan_report_counts_locates_and_names_the_stage():
    t = torch.ones(4, 5)
    t[1, 2] = t[3, 4] = float("nan")
    found, text = logged(check_and_log_nan_values, t, "w", "after update")
    assert found and "NaN values in w after update: 2 of 20 elements (10.0000%)" in text and "[[1, 2], [3, 4]]" in text
    cube = torch.zeros(2, 3, 4)
    cube[1, 2, 3] = float("nan")
    assert "[[1, 2, 3]]" in logged(check_and_log_nan_values, cube, "cube")[1]
    mixed = torch.tensor([float("nan"), float("inf"), 1.0])
    assert "1 of 3" in logged(check_and_log_nan_values, mixed, "mixed")[1]


def test_nan_report_lists_a_bounded_number_of_positions():
    t = torch.full((10, 10), float("nan"))
    found, text = logged(check_and_log_nan_values, t, "all")
    assert found and "100 of 100 elements (100.0000%)" in text and text.count("], [") == 19  # 20 positions by default
    assert logged(check_and_log_nan_values, t, "all", "", 3)[1].count("], [") == 2
    found, text = logged(check_and_log_nan_values, t, "all", "", 0)
    assert found and "first indices []" in text


def test_nan_scan_of_a_dict_names_each_entry():
    bad = torch.tensor([1.0, float("nan")])
    found, text = logged(check_and_log_nan_values, {"a": torch.ones(2), "b": bad}, "train")
    assert found and "train:b" in text and "train:a" not in text
    q = torch.tensor([1.0, float("nan")]).to(torch.float8_e4m3fn)
    assert logged(check_and_log_nan_values, q, "fp8")[0]


# ---- difference report -----------------------------------------------------------------------------
def test_agreement_within_and_beyond_tolerance():
    a = torch.linspace(0, 1, 12).reshape(3, 4)
    assert logged(compare_and_log_tensor_differences, a, a.clone(), "same")[0]
    assert logged(compare_and_log_tensor_differences, a, a + 1e-9, "close")[0]
    ok, text = logged(compare_and_log_tensor_differences, a, a + 1e-3, "far")
    assert not ok and "Tensor far differs in" in text
    assert logged(compare_and_log_tensor_differences, a, a + 1e-3, "loose", 1e-2, 0.0)[0]
    ok, text = logged(compare_and_log_tensor_differences, a, a + 1e-9, "exact", 0.0, 0.0, 20, True)
    assert not ok  # zero tolerance: bitwise


def test_shape_and_dtype_mismatches_are_reported_not_compared():
    a = torch.ones(2, 3)
    ok, text = logged(compare_and_log_tensor_differences, a, torch.ones(3, 2), "w")
    assert not ok and "Shape mismatch for w: (2, 3) vs (3, 2)" in text
    ok, text = logged(compare_and_log_tensor_differences, a, a.double(), "w")
    assert not ok and "Dtype mismatch for w" in text


def test_difference_report_names_elements_and_statistics():
    a = torch.zeros(4, 4)
    b = a.clone()
    b[0, 1], b[2, 3] = 0.5, -1.5
    ok, text = logged(compare_and_log_tensor_differences, a, b, "w")
    assert not ok and "differs in 2 of 16 elements: max abs 1.5, mean abs 0.125" in text
    assert "w[0, 1]: 0 vs 0.5" in text and "w[2, 3]: 0 vs -1.5" in text
    many = torch.ones(10, 10)
    ok, text = logged(compare_and_log_tensor_differences, torch.zeros(10, 10), many, "many", 1e-8, 1e-5, 5)
    assert not ok and "differs in 100 of 100" in text and text.count("  many[") == 5  # the list of positions is bounded


def test_pickled_cuda_tensors_name_their_gpu_by_uuid(monkeypatch):
    """The reduction patch swaps the device index for the GPU's UUID on the
    pickling side and finds the local index of that UUID on the other side,
    where the visible devices may be numbered differently."""
    from types import SimpleNamespace

    from torch.multiprocessing import reductions

    from awex_b200.utils import tensor_util

    uuids = ["GPU-aaaa", "GPU-bbbb", "GPU-cccc"]
    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda index: SimpleNamespace(uuid=uuids[index]))
    monkeypatch.setattr(torch.cuda, "device_count", lambda: len(uuids))
    rebuilt = []

    def fake_rebuild(*args):
        rebuilt.append(args)
        return "tensor"

    def fake_reduce(tensor):
        if tensor == "cpu tensor":
            return "rebuild_cpu", ("shared memory",)
        return reductions.rebuild_cuda_tensor, ("cls", (2,), (1,), 0, "storage_cls", torch.float32, 1, b"handle", 8, 0, False, b"ref", 0, b"event", True)

    monkeypatch.setattr(reductions, "rebuild_cuda_tensor", fake_rebuild)
    monkeypatch.setattr(reductions, "reduce_tensor", fake_reduce)
    monkeypatch.setattr(reductions, "init_reductions", lambda: None)
    try:
        tensor_util.monkey_patch_torch_reductions()
        patched = reductions.reduce_tensor
        tensor_util.monkey_patch_torch_reductions()  # a second call changes nothing
        assert reductions.reduce_tensor is patched
        rebuild, args = reductions.reduce_tensor("cuda tensor")
        assert args[6] == "GPU-bbbb" and args[7] == b"handle"
        assert reductions.reduce_tensor("cpu tensor") == ("rebuild_cpu", ("shared memory",))  # other reductions pass through
        # the receiving process numbers the same GPUs in another order
        uuids[:] = ["GPU-cccc", "GPU-bbbb", "GPU-aaaa"][::-1][1:] + ["GPU-aaaa"]  # bbbb is device 0 there
        assert rebuild(*args) == "tensor" and rebuilt[-1][6] == 0
        assert tensor_util.device_from_uuid(2) == 2  # plain indices pass through
        with pytest.raises(RuntimeError, match="no visible GPU"):
            tensor_util.device_from_uuid("GPU-zzzz")
    finally:
        for name in ("_awex_reduce_tensor", "_awex_rebuild_cuda_tensor"):
            if hasattr(reductions, name):
                delattr(reductions, name)
