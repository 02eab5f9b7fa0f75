"""CPU: host-side logic of the Python module (view metadata, errors, refusal to compute on CPU)."""
import numpy as np
import pytest

import aakaar_b200 as ak
from aakaar_b200 import _C


def cpu(shape):
    return ak.from_numpy(np.arange(int(np.prod(shape)), dtype=np.float32).reshape(shape), "cpu")


def test_api_surface_matches_reference_names():
    for name in ("matmul", "from_numpy", "set_tf32", "is_tf32_enabled", "synchronize", "no_grad", "mse_loss",
                 "add", "sub", "zero_grad_all", "is_grad_enabled"):
        assert hasattr(ak, name)
    for name in ("Tensor", "cuda_matmul", "cpu_matmul", "from_numpy", "_set_tf32_enabled", "_get_tf32_enabled",
                 "_synchronize", "empty_cache", "_allocator_stats", "_set_grad_enabled", "_is_grad_enabled",
                 "HAS_CUDA", "_sgd_step_fused", "_mse_fused", "is_available", "device_count",
                 "_set_cudnn_tf32_enabled", "_get_cudnn_tf32_enabled"):
        assert hasattr(_C, name), name
    assert hasattr(ak.nn, "Linear") and hasattr(ak.optim, "SGD") and hasattr(ak.losses, "MSELoss")


def test_view_metadata_follows_reference_semantics():
    t = cpu((2, 3, 4))
    assert t.shape == [2, 3, 4] and t.strides == [12, 4, 1] and t.size == 24 and t.is_contiguous()
    tt = t.transpose(1, 2)
    assert tt.shape == [2, 4, 3] and tt.strides == [12, 1, 4] and not tt.is_contiguous()
    assert t.T.shape == [2, 4, 3]
    assert t.transpose(-1, -2).strides == tt.strides
    s = t[1, 0:3:2, 1:]
    assert s.shape == [2, 3] and s.strides == [8, 1]
    np.testing.assert_array_equal(t.view([6, 4]).to_numpy(), t.to_numpy().reshape(6, 4))
    assert t.view([-1, 8]).shape == [3, 8]
    with pytest.raises(ValueError):
        tt.view([24])
    with pytest.raises(ValueError):
        t.view([5, 5])
    with pytest.raises(IndexError):
        t[5]


def test_tf32_flag_roundtrip_and_default():
    assert ak.is_tf32_enabled() is False
    ak.set_tf32(True)
    assert ak.is_tf32_enabled() is True
    ak.set_tf32(False)
    assert ak.is_tf32_enabled() is False


def test_no_grad_context():
    assert ak.is_grad_enabled()
    with ak.no_grad():
        assert not ak.is_grad_enabled()
    assert ak.is_grad_enabled()


def test_cpu_tensors_never_compute():
    a, b = cpu((2, 3)), cpu((3, 2))
    with pytest.raises(RuntimeError, match="no CPU"):
        ak.matmul(a, b)
    with pytest.raises(RuntimeError, match="no CPU matmul"):
        _C.cpu_matmul(a, b)
    with pytest.raises(RuntimeError):
        a + a
    with pytest.raises(RuntimeError):
        a.tanh()


def test_from_numpy_dtypes_and_missing_gpu():
    for dt, name in ((np.float32, "float32"), (np.float64, "float64"), (np.int32, "int32"), (np.int64, "int64")):
        t = ak.from_numpy(np.ones((2, 3), dtype=dt), "cpu")
        assert t.dtype == name and t.to_numpy().dtype == dt
    with pytest.raises(RuntimeError, match="unsupported dtype"):
        ak.from_numpy(np.ones((2, 2), dtype=np.float16), "cpu")
    with pytest.raises(RuntimeError, match="Only float32 currently supports gradients"):
        ak.from_numpy(np.ones((2, 2), dtype=np.float64), "cpu", requires_grad=True)
    if not ak.is_available():
        with pytest.raises(RuntimeError, match="no CPU path"):
            ak.from_numpy(np.ones((2, 2), dtype=np.float32), "cuda")


def test_dtype_enum_and_typed_constructor():
    from aakaar_b200 import _C
    assert [n for n in ("float32", "float64", "int32", "int64") if hasattr(_C.DType, n)] == ["float32", "float64", "int32", "int64"]
    t = _C.Tensor([2, 3], "cpu", _C.DType.int64)
    assert t.dtype == "int64" and t.shape == [2, 3] and t.to_numpy().dtype == np.int64
    assert _C.Tensor([4], "cpu").dtype == "float32"


def test_sgd_argument_check():
    with pytest.raises(ValueError):
        ak.optim.SGD([], nesterov=True)


def test_conv_callers_argument_checks_without_gpu():
    # shape logic and error behaviour of the convolution callers run on the host; computing needs the GPU
    x = ak.from_numpy(np.ones((2, 3, 8), dtype=np.float32), "cpu")
    w = ak.from_numpy(np.ones((4, 3, 9), dtype=np.float32), "cpu")
    with pytest.raises(ValueError, match="computed output length"):
        ak.conv1d(x, w)                                   # kernel longer than the input
    with pytest.raises(ValueError, match="expected input of shape"):
        ak.im2col_1d(ak.from_numpy(np.ones((2, 3), dtype=np.float32), "cpu"), 3, 1, 0, 1, 1)
    with pytest.raises(ValueError, match="expected input of shape"):
        ak.im2col_2d(x, 3, 3, 1, 1, 0, 0, 1, 1, 1, 1)
    conv = ak.nn.Conv1d(3, 4, 3, device="cpu")
    assert conv.weight.shape == [4, 3, 3] and conv.bias.shape == [1, 4, 1] and len(conv.parameters()) == 2
    with pytest.raises(ValueError, match="input channels"):
        conv(ak.from_numpy(np.ones((2, 5, 8), dtype=np.float32), "cpu"))
    with pytest.raises(RuntimeError):
        conv(x)                                           # CPU tensors do not compute
    with pytest.raises(RuntimeError, match="float32 only"):
        ak.nn.Conv2d(3, 4, 3, device="cpu", dtype="float64")


def test_muon_and_fusion_switch_exist():
    from aakaar_b200 import _C
    _C._set_backward_fusion(False)
    _C._set_backward_fusion(True)
    opt = ak.optim.Muon([ak.from_numpy(np.ones((2, 2), dtype=np.float32), "cpu", requires_grad=True)])
    opt.step()          # no gradients yet: nothing to do
    opt.zero_grad()
    with pytest.raises(RuntimeError):
        _C.matmul_axpby(ak.from_numpy(np.ones((2, 2), dtype=np.float32), "cpu"),
                        ak.from_numpy(np.ones((2, 2), dtype=np.float32), "cpu"), 1.0, 0.0, None)
