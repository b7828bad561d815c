"""The allocation-free batch-1 entry point (cbl_gemv_l8_static), called through the C ABI, against the
regular entry point (cbl_gemv_l8) on the same inputs, twice in a row.

Collected last on purpose: the scratch array it uses is shared by the whole process, so running it
after everything else also shows that earlier work leaves nothing behind that disturbs it."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import cbl_oracle as orc

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_workspace_entry_on_two_consecutive_calls():
    from quantexperiments_b200 import _lib
    from quantexperiments_b200.kernels import DeviceMatrix, L8Matrix, l8_workspace
    lib = _lib.lib
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    for R, C, books in ((4864, 896, 1), (2051, 1024, 2)):
        m = orc.synth_matrix(R, C, seed=R, books=books)
        dm = DeviceMatrix(t(m["words"][0]), t(m["table"][0]), t(m["row_scale"]), K=4096, d=8, C=C,
                          tags2=t(m["words"][1]) if books == 2 else None, table2=t(m["table"][1]) if books == 2 else None)
        l8 = L8Matrix(dm)
        st = l8.struct()
        ref_w = orc.synth_decode(m)
        g = torch.Generator().manual_seed(C)
        stream = torch.cuda.current_stream().cuda_stream
        for call in range(2):                       # two calls in a row: the second finds the first one's leftovers
            x = torch.randn(C, generator=g).bfloat16().cuda()
            y_ws = torch.full((R,), float("nan"), device="cuda")
            y_st = torch.full((R,), float("nan"), device="cuda")
            ws = l8_workspace(dm.device, R)
            rc = lib.cbl_gemv_l8(ctypes.byref(st), x.data_ptr(), _lib.BF16, y_ws.data_ptr(), _lib.F32, ws.data_ptr(), stream)
            assert rc == _lib.OK
            before = torch.cuda.memory_allocated()
            rc = lib.cbl_gemv_l8_static(ctypes.byref(st), x.data_ptr(), _lib.BF16, y_st.data_ptr(), _lib.F32, stream)
            assert rc == _lib.OK
            assert torch.cuda.memory_allocated() == before
            torch.cuda.synchronize()
            yref = orc.linear_ref(x.float().cpu().numpy()[None], ref_w)[0]
            assert orc.max_rel_err(y_st.cpu().numpy(), y_ws.cpu().numpy()) < 1e-5      # same kernel, reduction order may differ
            assert orc.max_rel_err(y_st.cpu().numpy(), yref) < 1e-3
        # the Python wrapper takes the same path
        y2 = l8.run_static(x, torch.empty(R, device="cuda"))
        assert orc.max_rel_err(y2.cpu().numpy(), yref) < 1e-3


def test_static_scratch_entry_rejects_matrices_beyond_its_fixed_capacity():
    from quantexperiments_b200 import _lib
    lib = _lib.lib
    cap = lib.cbl_gemv_l8_static_max_rows()
    assert cap == 65536
    big = _lib.L8(R=cap + 4, C=64, books=1, ntile=1, Rpad=cap + 4)
    x = torch.zeros(64, device="cuda", dtype=torch.bfloat16)
    y = torch.zeros(cap + 4, device="cuda")
    rc = lib.cbl_gemv_l8_static(ctypes.byref(big), x.data_ptr(), _lib.BF16, y.data_ptr(), _lib.F32, None)
    assert rc == _lib.EUNSUPPORTED
    assert b"unsupported" in lib.cbl_status_string(rc)
