"""CPU-only checks of the drop-in boundary: the library loads, exports every symbol the header declares, the header
covers the reference's whole backend interface, and calls that cannot run without a GPU fail loudly instead of
falling back to anything."""
import ctypes
import json
import os

from minml_b200 import _abi

HERE = os.path.dirname(__file__)


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_abi.LIBRARY)
    names = _abi.declared_symbols()
    assert len(names) == len(set(names))
    for name in names:
        assert hasattr(lib, name), name


def test_header_covers_the_reference_interface():
    # tests/golden/cuda_backend_symbols.json lists the 113 functions of the reference's include/minml/backend/cuda_backend.h
    wanted = json.load(open(os.path.join(HERE, "golden", "cuda_backend_symbols.json")))["symbols"]
    assert len(wanted) == 113
    declared = set(_abi.declared_symbols())
    assert [w for w in wanted if w not in declared] == []


def test_descriptor_layouts():
    assert ctypes.sizeof(_abi.mlTensor_t) == 40  # pointer, dtype, rank, int[6]
    assert ctypes.sizeof(_abi.mlShape_t) == 28
    assert ctypes.sizeof(_abi.mlQuantizationData_t) == 8


def test_no_device_means_no_context():
    lib = _abi.load()
    if lib.cuda_get_number_of_devices() > 0:
        return
    lib.mb200_clear_last_error(None)
    assert not lib.cuda_create_context(0)
    assert b"out of range" in lib.mb200_get_last_error(None)
    assert not lib.cuda_supports_type(0, _abi.DTYPE_FLOAT16)
    lib.mb200_clear_last_error(None)


def test_stub_records_not_implemented_without_a_context():
    lib = _abi.load()
    lib.mb200_clear_last_error(None)
    t = _abi.mlTensor_t()
    lib.cuda_hash_routing(None, t, t)
    assert b"not implemented" in lib.mb200_get_last_error(None)
    lib.mb200_clear_last_error(None)


def test_tensor_on_another_device_is_refused_on_the_host():
    """A tensor that lives on cuda:0 must not reach a context of cuda:1: the Python mirror raises before any launch.  Checked
    here with stand-ins (no GPU needed): the test is about the host-side guard, not about device memory."""
    import types

    import pytest

    from minml_b200 import backend as B

    class FakeTensor:
        def __init__(self, index):
            self.is_cuda = True
            self.device = types.SimpleNamespace(index=index)
            self.shape = (2, 3)
            self.dtype = None

        def is_contiguous(self):
            return True

        def data_ptr(self):
            return 256

    fake_ctx = types.SimpleNamespace(device_index=1)
    assert B.ptr(FakeTensor(1), fake_ctx).value == 256
    assert B.ptr(None, fake_ctx) is None
    with pytest.raises(B.BackendError, match="cuda:0 passed to a context of cuda:1"):
        B.ptr(FakeTensor(0), fake_ctx)
    with pytest.raises(B.BackendError, match="cuda:0 passed to a context of cuda:1"):
        B.desc(FakeTensor(0), fake_ctx)
