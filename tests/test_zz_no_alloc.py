"""The allocation-free sort entry point against the regular one.

Some users of the library cannot allocate device memory where they call it (their own
pool owns the device heap, or they run inside another framework's budget), so
``flymoe_moe_sorting_noalloc`` keeps its scratch in an array built into the library.
This file is collected last on purpose: a run that stops at the first failure has then
already executed every other test.  It must pass alone in a fresh process and after the
rest of the suite; both calls below go straight through the C ABI.
"""
import pytest
import torch

from flydsl_b200 import _lib
from tests import helpers as hp

pytestmark = pytest.mark.gpu


def _outputs(T, E, k, unit):
    cap = T * k + E * unit - k
    d = "cuda"
    return [torch.full((cap,), -3, dtype=torch.int32, device=d), torch.full((cap,), -3.0, dtype=torch.float32, device=d),
            torch.full(((cap + unit - 1) // unit,), -3, dtype=torch.int32, device=d),
            torch.full((2,), -3, dtype=torch.int32, device=d)]


def _call(fn_name, ids, w, outs, buf, mask, T, E, k, unit, ws=None):
    lib = _lib.load()
    s = torch.cuda.current_stream().cuda_stream
    common = [ids.data_ptr(), w.data_ptr(), outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr(),
              outs[3].data_ptr(), buf.data_ptr(), buf.numel() * buf.element_size(), _lib.ptr(mask)]
    if fn_name == "noalloc":
        rc = lib.flymoe_moe_sorting_noalloc(*common, T, E, k, unit, s)
    else:
        rc = lib.flymoe_moe_sorting(*common, _lib.ptr(ws), 0 if ws is None else ws.numel(), T, E, k, unit, s)
    _lib.check(rc, fn_name)


@pytest.mark.parametrize("T,E,k,unit,masked", [(64, 256, 8, 32, False), (4096, 256, 8, 128, False),
                                               (16384, 256, 8, 128, True), (3000, 64, 6, 16, False)])
def test_noalloc_sort_matches_regular_entry_point(T, E, k, unit, masked):
    lib = _lib.load()
    need = lib.flymoe_moe_sorting_workspace_elems(T, E, k, unit)
    assert need <= lib.flymoe_moe_sorting_noalloc_max_elems()
    mask = None
    if masked:
        mask = (torch.arange(E) % 3 != 0).to(torch.int32).cuda()
    for call in range(2):                      # two calls in a row share the built-in scratch
        ids, w = hp.fast_sort_inputs(T, E, k, 1000 + call, device="cuda")
        ws = torch.empty(max(need, 1), dtype=torch.int32, device="cuda")
        ref, got = _outputs(T, E, k, unit), _outputs(T, E, k, unit)
        buf_ref = torch.ones((T, 16), dtype=torch.float32, device="cuda")
        buf_got = torch.ones((T, 16), dtype=torch.float32, device="cuda")
        _call("regular", ids, w, ref, buf_ref, mask, T, E, k, unit, ws)
        _call("noalloc", ids, w, got, buf_got, mask, T, E, k, unit)
        torch.cuda.synchronize()
        R = int(ref[3][0])
        assert torch.equal(got[3], ref[3])
        assert torch.equal(got[0][:R], ref[0][:R])
        assert torch.equal(got[1][:R].view(torch.int32), ref[1][:R].view(torch.int32))
        assert torch.equal(got[2], ref[2])
        assert float(buf_got.abs().sum()) == 0.0 and float(buf_ref.abs().sum()) == 0.0


def test_noalloc_sort_rejects_oversized_problem():
    lib = _lib.load()
    T, E, k, unit = 1 << 20, 1024, 8, 32       # needs 16384 * 1024 + 1024 int32 of scratch
    assert lib.flymoe_moe_sorting_workspace_elems(T, E, k, unit) > lib.flymoe_moe_sorting_noalloc_max_elems()
    one = torch.zeros(8, dtype=torch.int32, device="cuda")
    rc = lib.flymoe_moe_sorting_noalloc(one.data_ptr(), one.data_ptr(), one.data_ptr(), one.data_ptr(),
                                        one.data_ptr(), one.data_ptr(), None, 0, None, T, E, k, unit,
                                        torch.cuda.current_stream().cuda_stream)
    assert rc == -4
    assert b"built-in array" in lib.flymoe_last_error()
