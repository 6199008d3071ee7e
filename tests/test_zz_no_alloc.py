"""The allocation-free weight-prep entry point against the ordinary one (collected last on purpose).

Some callers of this library cannot allocate device memory when compression fires: a serving worker
whose free HBM has all gone to the KV-cache pool, or a hook inside the engine's step loop where a
cudaMalloc would synchronise the device.  ``triattn_prep_weights_noalloc`` serves them from a scratch
array built into the library.  This test calls it through the C ABI twice in a row (the second call
finds the first call's leftovers in the shared scratch) and compares with ``triattn_prep_weights``.
"""
from __future__ import annotations

import ctypes

import pytest
import torch

from triattention_b200 import _native, ops
import synth

pytestmark = pytest.mark.gpu


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _stats(dev, L, Hq, D, seed):
    gen = torch.Generator().manual_seed(seed)
    inv_freq = synth.rope_inv_freq(D, 1e6)
    st = synth.make_stats(L, Hq, D, inv_freq, gen)
    fs = (0.5 + torch.rand((L, Hq, D // 2), generator=gen))
    offsets = torch.tensor([float(2 ** i) for i in range(17)])
    return ops.DeviceStats(st.q_mean_real.to(dev), st.q_mean_imag.to(dev), st.q_abs_mean.to(dev), fs.to(dev),
                           inv_freq.to(dev), offsets.to(dev))


def _noalloc(lib, st, rs, agg, flags, out):
    L, Hq, F = st.num_layers, st.num_heads, st.num_freqs
    return lib.triattn_prep_weights_noalloc(
        _ptr(st.q_mean_real), _ptr(st.q_mean_imag), _ptr(st.q_abs_mean), _ptr(st.freq_scale_sq), _ptr(st.omega),
        _ptr(st.offsets), _ptr(rs), L, int(rs.numel()), Hq, F, int(st.offsets.numel()), agg, flags, _ptr(out),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


def test_noalloc_prep_matches_regular_entry_twice_in_a_row():
    lib = _native.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    st = _stats(dev, 3, 8, 128, 77)
    calls = [
        (torch.tensor([4096, 33000, 7, 100001], dtype=torch.int32, device=dev), _native.OFFSETS_MEAN, 0),
        # second call: other round starts, per-offset rows and an ablation flag; the scratch still holds call 1's tables
        (torch.tensor([123, 65536], dtype=torch.int32, device=dev), _native.OFFSETS_MAX, _native.FLAG_DISABLE_MLR),
        (torch.tensor([4096, 33000, 7, 100001], dtype=torch.int32, device=dev), _native.OFFSETS_MEAN, 0),
    ]
    for rs, agg, flags in calls:
        expect = ops.prep_weights(st, rs, agg, flags)            # existing entry point, caller-allocated scratch
        got = torch.full_like(expect, float("nan"))              # outputs are still the caller's
        rc = _noalloc(lib, st, rs, agg, flags, got)
        assert rc == _native.OK, _native.status_string(rc)
        torch.cuda.synchronize()
        # same kernels on the same inputs: the tolerance of the score tests (1e-3 relative) is met exactly
        assert torch.equal(got, expect)
        assert torch.allclose(got, expect, rtol=1e-3, atol=0.0)


def test_noalloc_prep_rejects_sizes_beyond_its_scratch():
    lib = _native.load()
    dev = torch.device("cuda", 0)
    st = _stats(dev, 1, 2, 128, 78)
    # MAX aggregation needs B*2*17*64 floats: 31 requests exceed the 65536-float scratch, 30 fit
    rs = torch.zeros(31, dtype=torch.int32, device=dev)
    out = torch.zeros((1, 31, 2, 35, 64), dtype=torch.float32, device=dev)
    assert _noalloc(lib, st, rs, _native.OFFSETS_MAX, 0, out) == _native.ERR_LIMIT_EXCEEDED
    assert "maximum" in _native.status_string(_native.ERR_LIMIT_EXCEEDED)
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0  # nothing was launched
    assert _noalloc(lib, st, rs[:30], _native.OFFSETS_MAX, 0, out) == _native.OK
    torch.cuda.synchronize()
