"""The host-CPU AdamWBF16 (C++ / OpenMP) against the bit-exact Python twin of the device kernel."""

import ctypes

import pytest
import torch

from halo_b200.ops import _lib
from halo_b200.optim.adamw_bf16 import SR_KEY, adamw_bf16_step_reference, param_name_hash


@pytest.mark.parametrize("n", [1, 7, 1024, 4099, 300001])
@pytest.mark.parametrize("scale", [None, 0.37])
def test_host_step_is_bit_identical_to_the_reference(n, scale):
    torch.manual_seed(n)
    p = torch.randn(n).bfloat16()
    g = (torch.randn(n) * 0.1).bfloat16()
    m = (torch.randn(n) * 0.01).bfloat16()
    v = (torch.rand(n) * 1e-3).bfloat16()
    kw = dict(beta1=0.9, beta2=0.999, step_size=1e-3 / (1 - 0.9**3), bc2_sqrt=(1 - 0.999**3) ** 0.5, eps=1e-8,
              wd_factor=1.0 - 1e-3 * 0.01)
    name_hash = param_name_hash("layers.3.mlp.experts_gate_up")
    rp, rm, rv = p.clone(), m.clone(), v.clone()
    adamw_bf16_step_reference(rp, g, rm, rv, key=SR_KEY, step=3, name_hash=name_hash, grad_scale=scale, **kw)
    L = _lib.host_lib()
    u16 = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    for threads in (1, 3):
        hp, hm, hv = p.clone(), m.clone(), v.clone()
        rc = L.halo_host_adamw_bf16(
            u16(hp), u16(g), u16(hm), u16(hv), ctypes.c_longlong(n), ctypes.c_ulonglong(name_hash),
            ctypes.c_ulonglong(SR_KEY), ctypes.c_ulonglong(3), ctypes.c_float(kw["beta1"]), ctypes.c_float(kw["beta2"]),
            ctypes.c_float(kw["step_size"]), ctypes.c_float(kw["bc2_sqrt"]), ctypes.c_float(kw["eps"]),
            ctypes.c_float(kw["wd_factor"]), ctypes.c_float(scale if scale is not None else 1.0),
            ctypes.c_int(0 if scale is None else 1), ctypes.c_int(threads))
        assert rc == 0
        assert torch.equal(hm.view(torch.int16), rm.view(torch.int16)), "first moment"
        assert torch.equal(hv.view(torch.int16), rv.view(torch.int16)), "second moment"
        assert torch.equal(hp.view(torch.int16), rp.view(torch.int16)), "weights"
