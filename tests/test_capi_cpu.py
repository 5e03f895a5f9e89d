"""CPU tests of the boundary: the C-ABI library builds, loads and exports every declared symbol;
host-side argument checks that need no device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tnn_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tnn_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(tnn_lib):
    lib = ctypes.CDLL(os.path.join(ROOT, "tiny-dpcpp-nn_b200", "libtnn_b200.so"))
    declared = _declared_symbols()
    assert len(declared) >= 30
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/tnn_b200.h but not exported"


def test_python_binding_covers_header(tnn_lib):
    assert set(_declared_symbols()) == set(tnn_lib.exported_symbols())


def test_argument_errors_need_no_device(tnn_lib):
    lib = tnn_lib.load()
    h = ctypes.c_void_p()
    # width outside {16, 32, 64, 128}: Network.h:163-164
    assert lib.tnn_network_create(64, 64, 4, 0, 8, 48, 0, 1, ctypes.byref(h)) != 0
    assert b"power of 2" in lib.tnn_last_error()
    # unsupported activation: SwiftNetMLP.h:281-288
    assert lib.tnn_network_create(64, 64, 4, 7, 8, 64, 0, 1, ctypes.byref(h)) != 0
    # input wider than the network: Network.h:142-147
    assert lib.tnn_network_create(65, 64, 4, 0, 8, 64, 0, 1, ctypes.byref(h)) != 0
    assert b"Input width" in lib.tnn_last_error()
    # no hidden layer: Network.h:156-160
    assert lib.tnn_network_create(64, 64, 0, 0, 8, 64, 0, 1, ctypes.byref(h)) != 0
    # encodings: bad JSON, unknown type, missing keys (encoding_factory.h:28-45, 113-125)
    e = ctypes.c_void_p()
    assert lib.tnn_encoding_create(b"not json", 0, ctypes.byref(e)) != 0
    assert lib.tnn_encoding_create(b'{"otype": "Nope"}', 0, ctypes.byref(e)) != 0
    assert b"Unknown encoding type" in lib.tnn_last_error()
    assert lib.tnn_encoding_create(b'{"n_levels": 4}', 0, ctypes.byref(e)) != 0
    # frequency encoding (test/doctest_encodings.cpp:357-404): missing / zero / negative n_frequencies, zero input
    # dims, padded width below the natural width
    for cfg, pad in ((b'{"otype": "Frequency", "n_dims_to_encode": 1}', 0),
                     (b'{"otype": "Frequency", "n_dims_to_encode": 1, "n_frequencies": 0}', 0),
                     (b'{"otype": "Frequency", "n_dims_to_encode": 1, "n_frequencies": -1}', 0),
                     (b'{"otype": "Frequency", "n_dims_to_encode": 0, "n_frequencies": 1}', 0),
                     (b'{"otype": "Frequency", "n_dims_to_encode": 1, "n_frequencies": 1}', 1)):
        assert lib.tnn_encoding_create(cfg, pad, ctypes.byref(e)) != 0, cfg
    # spherical harmonics (spherical_harmonics.h:18-26, encoding_factory.h:55-72): 3-D only, degree in [1, 8]
    for cfg, msg in ((b'{"otype": "SphericalHarmonics", "n_dims_to_encode": 2, "degree": 4}', b"3D directions"),
                     (b'{"otype": "SphericalHarmonics", "n_dims_to_encode": 3, "degree": 9}', b"degree > 0 and <= 8"),
                     (b'{"otype": "SphericalHarmonics", "n_dims_to_encode": 3, "degree": 0}', b"degree > 0 and <= 8"),
                     (b'{"otype": "SphericalHarmonics", "n_dims_to_encode": 3}', b"misses degree")):
        assert lib.tnn_encoding_create(cfg, 0, ctypes.byref(e)) != 0
        assert msg in lib.tnn_last_error(), (cfg, lib.tnn_last_error())
    # fp16 networks are accepted (argument checks come first either way)
    assert lib.tnn_network_create(64, 64, 4, 0, 8, 48, 1, 1, ctypes.byref(h)) != 0
    assert b"power of 2" in lib.tnn_last_error()
    assert lib.tnn_network_create(64, 64, 4, 0, 8, 64, 2, 1, ctypes.byref(h)) != 0
    assert b"Only fp16 and bf16" in lib.tnn_last_error()


def test_no_device_means_loud_failure(tnn_lib):
    """Without a CUDA device create must fail with a message - there is no CPU path to fall back to."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    lib = tnn_lib.load()
    h = ctypes.c_void_p()
    assert lib.tnn_network_create(64, 64, 4, 0, 8, 64, 0, 1, ctypes.byref(h)) != 0
    assert len(lib.tnn_last_error()) > 0
    e = ctypes.c_void_p()
    assert lib.tnn_encoding_create(b'{"otype": "Identity", "n_dims_to_encode": 2, "scale": 1.0, "offset": 0.0}', 0,
                                   ctypes.byref(e)) != 0


def test_python_package_names():
    import tiny_dpcpp_nn

    for name in ("Network", "Encoding", "NetworkWithInputEncoding", "free_temporary_memory"):
        assert hasattr(tiny_dpcpp_nn, name)
    from tiny_dpcpp_nn.modules import to_packed_layout_coord, from_packed_layout_coord

    for idx in range(64):
        assert from_packed_layout_coord(to_packed_layout_coord(idx, 8, 8), 8, 8) == idx
