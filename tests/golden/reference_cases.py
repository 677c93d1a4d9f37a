"""Known-answer cases of the reference's own test-suite for the padding / mask path, as data.

Each case carries the literal inputs and expected outputs that the reference asserts in
test/test_nested_tensor_masking.py (line ranges given per case).  They pin the CPU oracle
(tests/test_oracle_golden.py) and are replayed against the CUDA path (tests/test_golden_gpu.py).
"""
import torch

T = torch.tensor

# ---- to_tensor_mask: (constituents, mask_dim, expected tensor, expected mask)   [:11-142]
TO_TENSOR_MASK = [
    # test_empty_nt :11-16
    ("empty_nt", [], None, T([0]), T(False)),
    # test_single_scalar :26-49
    ("single_scalar", [T(1, dtype=torch.uint8)], None, T([1], dtype=torch.uint8), T(True)),
    ("single_scalar_md0", [T(1, dtype=torch.uint8)], 0, T([1], dtype=torch.uint8), T(True)),
    ("single_scalar_md1", [T(1, dtype=torch.uint8)], 1, T([1], dtype=torch.uint8), T([True])),
    # test_single_tensor :80-103
    ("single_tensor", [T([1])], None, T([[1]]), T(True)),
    ("single_tensor_md0", [T([1])], 0, T([[1]]), T(True)),
    ("single_tensor_md1", [T([1])], 1, T([[1]]), T([True])),
    ("single_tensor_md2", [T([1])], 2, T([[1]]), T([[True]])),
    # test_multi_tensor :105-131
    ("multi_tensor", [T([1]), T([2]), T([3])], None, T([[1], [2], [3]]), T(True)),
    ("multi_tensor_md0", [T([1]), T([2]), T([3])], 0, T([[1], [2], [3]]), T(True)),
    ("multi_tensor_md1", [T([1]), T([2]), T([3])], 1, T([[1], [2], [3]]), T([True, True, True])),
    ("multi_tensor_md2", [T([1]), T([2]), T([3])], 2, T([[1], [2], [3]]), T([[True], [True], [True]])),
]

# ---- to_tensor_mask error cases: (constituents, mask_dim, message regex)
TO_TENSOR_MASK_ERRORS = [
    # test_empty_tensor :19-24
    ("empty_tensor", [T([])], None, "Empty tensors are not yet supported."),
    # test_single_scalar :46-49
    ("single_scalar_md2", [T(1, dtype=torch.uint8)], 2,
     "Requested mask dimension 2 is bigger than dimension 1 of given NestedTensor."),
    # test_single_tensor :100-103
    ("single_tensor_md3", [T([1])], 3,
     "Requested mask dimension 3 is bigger than dimension 2 of given NestedTensor."),
    # test_mask_dim_too_small_error :133-141
    ("too_small", [T([1, 2]), T([3, 4, 5, 6])], 1, "Mask dimension is too small to represent data tensor."),
]

# ---- nested_tensor_from_tensor_mask: (tensor, mask, nested_dim, expected constituents)   [:146-452]
FROM_TENSOR_MASK = [
    # test_ntftm_empty3 :189-194
    ("empty3", T([0]), T(False), 1, []),
    # test_ntftm_single_scalar_mask_false :211-216
    ("single_scalar_mask_false", T([1], dtype=torch.uint8), T(False), 1, []),
    # test_ntftm_single_scalar :224-243
    ("single_scalar_true", T([1.0]), T(True), 1, [T(1.0)]),
    ("single_scalar_true1", T([1.0]), T([True]), 1, [T(1.0)]),
    ("single_scalar_extra_dim", T([[1.0]]), T(True), 1, [T([1.0])]),
    # test_ntftm_multi_scalars :245-278
    ("multi_scalars", T([1, 2, 3]), T(True), 1, [T(1), T(2), T(3)]),
    ("multi_scalars_extra_dim", T([[1, 2, 3]]), T(True), 1, [T([1, 2, 3])]),
    # test_ntftm_multi_tensor_scalar_true_mask :292-313
    ("multi_tensor_scalar_true", T([[1], [2], [3]]), T(True), 1, [T([1]), T([2]), T([3])]),
    ("multi_tensor_scalar_true_extra", T([[[1]], [[2]], [[3]]]), T(True), 1, [T([[1]]), T([[2]]), T([[3]])]),
    # test_ntftm_multi_tensor_true_mask :315-352
    ("true_mask3", T([[[1.0]], [[2.0]], [[3.0]]]), T([[[True]], [[True]], [[True]]]), 1,
     [T([[1.0]]), T([[2.0]]), T([[3.0]])]),
    ("true_mask2", T([[[1.0]], [[2.0]], [[3.0]]]), T([[True], [True], [True]]), 1,
     [T([[1.0]]), T([[2.0]]), T([[3.0]])]),
    ("true_mask1", T([[[1.0]], [[2.0]], [[3.0]]]), T([True, True, True]), 1,
     [T([[1.0]]), T([[2.0]]), T([[3.0]])]),
    ("true_mask0", T([[[1.0]], [[2.0]], [[3.0]]]), T(True), 1, [T([[1.0]]), T([[2.0]]), T([[3.0]])]),
    # test_ntftm_single_tensor_all_false_mask :354-363
    ("single_all_false", T([[1]]), T([False]), 1, []),
    ("single_all_false3", T([[1, 2, 3]]), T([False]), 1, []),
    # test_ntftm_multi_tensor_all_false_mask :365-381 (first case)
    ("multi_all_false", T([[[1], [2], [3]]]), T([False]), 1, []),
    # test_ntftm_multi_tensor_all_false_mask2 :383-390
    ("multi_all_false2", T([[[1], [2], [3]]]), T([[[False], [False], [False]]]), 1,
     [torch.empty((3, 0), dtype=torch.int64)]),
    # test_ntgtm_multi_scalar_mix_mask :392-401
    ("scalar_mix", T([1.0, 2.0, 3.0, 4.0]), T([True, False, False, True]), 1, [T(1.0), T(4.0)]),
    # test_ntgtm_multi_tensor_mix_mask :403-412
    ("tensor_mix", T([[1.0], [2.0], [3.0], [4.0]]), T([True, False, False, True]), 1, [T([1.0]), T([4.0])]),
    # test_ntgtm_scalar_with_empty_mix_mask :414-423
    ("scalar_with_empty_mix", T([[0.0], [11.0]]), T([False, True]), 1, [T([11.0])]),
    # test_ntftm_test_multi_tensor_mix_mask :425-437
    ("mix_mask", T([[1.0, 2.0, 3.0], [4.0, 0.0, 0.0]]), T([[True, True, True], [True, False, False]]), 1,
     [T([1.0, 2.0, 3.0]), T([4.0])]),
    # test_ntftm_test_multi_tensor_mix_mask2 :439-452
    ("mix_mask2", T([[[1.0, 2.0, 3.0]], [[4.0, 0.0, 0.0]]]),
     T([[[True, True, True]], [[True, False, False]]]), 1, [T([[1.0, 2.0, 3.0]]), T([[4.0]])]),
]

# ---- argument errors of nested_tensor_from_tensor_mask   [:146-222, :218-222]
FROM_TENSOR_MASK_ERRORS = [
    ("nested_dim_0", T([]), T([]), 0, "Nested dimension can't be 0."),
    ("data_empty", T([]), T([True]), 1, "Data tensor can't be emtpy if a mask has values."),
    ("mask_empty", T([1]), T([]), 1, "Mask tensor can't be emtpy if a data tensor has values."),
    ("scalar", T(1), T(True), 1, "Can't construct nested tensor from a scalar."),
]

# ---- test_to_padded_tensor :454-477: explicit round trip and padding = -10
ROUNDTRIP_DATA = T(
    [[[0.8413, 0.7325, 0.0000, 0.0000],
      [0.0000, 0.0000, 0.0000, 0.0000],
      [0.0000, 0.0000, 0.0000, 0.0000]],
     [[0.6334, 0.5473, 0.3273, 0.0564],
      [0.3023, 0.6826, 0.3519, 0.1804],
      [0.8431, 0.1645, 0.1821, 0.9185]]])
ROUNDTRIP_MASK = T(
    [[[True, True, False, False],
      [False, False, False, False],
      [False, False, False, False]],
     [[True, True, True, True],
      [True, True, True, True],
      [True, True, True, True]]])
ROUNDTRIP_PADDING = -10
