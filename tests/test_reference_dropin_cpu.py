"""The UNMODIFIED reference tmq/tmq.py running on top of this library's entropy coder.

The reference binds its native helper with `from .tmq_native import ...` (tmq/tmq.py:28-46).  Here that module name is
bound to a stand-in whose compress_ternary / decompress_ternary are tmq_b200.codec's (host code inside libtmq_b200.so)
while the packer stays the reference's own (this library packs on the GPU, and this test runs without one).  The
reference's compressed_state_dict(strong=True) / load_compressed_state_dict round trip must then produce byte-identical
streams and identical packed weights to the reference's own helper.

Needs the reference checkout (TMQ_REFERENCE_DIR, or a checkout beside this repository) and oracle/_ref/tmq_native.so;
skipped elsewhere.  The CUDA half of the same drop-in (tmq_cuda -> tmq_b200.ops) needs a GPU and the checkout on one
machine, which no test box here offers; tests/test_reference_kernels_gpu.py covers it operator by operator instead."""
import contextlib
import io
import os
import sys
import types

import pytest
import torch
from torch import nn

from oracle import build_ref


@pytest.fixture()
def reference_with(request):
    if not os.path.isfile(os.path.join(build_ref.REFERENCE, "tmq", "tmq.py")):
        pytest.skip("reference checkout not present")
    native = build_ref.load_native()
    if native is None:
        pytest.skip("oracle/_ref/tmq_native.so not built")

    def load(native_module):
        for k in [k for k in sys.modules if k == "tmq" or k.startswith("tmq.")]:
            del sys.modules[k]
        sys.modules["tmq.tmq_native"] = native_module
        sys.path.insert(0, build_ref.REFERENCE)
        try:
            with contextlib.redirect_stdout(io.StringIO()):
                import tmq as ref
        finally:
            sys.path.remove(build_ref.REFERENCE)
        assert ref.NATIVE_EXT_AVAILABLE
        return ref

    yield native, load
    for k in [k for k in sys.modules if k == "tmq" or k.startswith("tmq.")]:
        del sys.modules[k]


def _model():
    torch.manual_seed(3)
    return nn.Sequential(nn.Conv2d(3, 20, 3, padding=1), nn.ReLU(), nn.Flatten(), nn.Linear(20 * 6 * 6, 37))


def _strong_dict(ref):
    model = _model()
    ctrl = ref.QuantizationControl()
    with contextlib.redirect_stdout(io.StringIO()):
        ref.quantize_model(model, ctrl)
    g = torch.Generator().manual_seed(11)
    with torch.no_grad():
        for node in ctrl._registry.values():
            node.weight.copy_(torch.randint(-1, 2, node.weight.shape, generator=g).float())
    ref.compressed_state_dict(model, strong=False)        # the reference's own packer
    state = ref.compressed_state_dict(model, strong=True)  # compress_ternary(packed, shape, True)
    fresh = _model()
    with contextlib.redirect_stdout(io.StringIO()):
        ref.quantize_model(fresh, ref.QuantizationControl())
    ref.load_compressed_state_dict(fresh, state)            # decompress_ternary
    packed = {k: v.detach().clone() for k, v in fresh.state_dict().items() if v.dtype == torch.int32}
    streams = {k: v.detach().clone() for k, v in state.items() if v.dtype == torch.int8}
    return streams, packed


def test_reference_state_dict_round_trip_on_this_librarys_coder(reference_with):
    native, load = reference_with
    from tmq_b200 import codec
    want_streams, want_packed = _strong_dict(load(native))
    stand_in = types.ModuleType("tmq_native")
    stand_in.compactify_ternary = native.compactify_ternary
    stand_in.expand_ternary = native.expand_ternary
    stand_in.compress_ternary = codec.compress_ternary
    stand_in.decompress_ternary = codec.decompress_ternary
    got_streams, got_packed = _strong_dict(load(stand_in))
    assert len(want_streams) == 2 and set(got_streams) == set(want_streams)
    for k in want_streams:
        assert torch.equal(got_streams[k], want_streams[k]), k
    assert set(got_packed) == set(want_packed) and len(want_packed) == 2
    for k in want_packed:
        assert torch.equal(got_packed[k], want_packed[k]), k
