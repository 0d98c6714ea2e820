"""The bounded-wait abort path, executed once on the GPU without any fault: a one-CTA kernel waits on
a barrier nobody arrives on, gives up after its (sub-millisecond) limit, raises the CTA's abort flag,
and the second warp -- waiting with the library's default limit -- leaves through that flag.  The
host then reads the status word, and `_lib.check_status` is shown to see both status words."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("parked", [0, 1])
@pytest.mark.parametrize("limit_us", [50, 800])
def test_wait_gives_up_and_reports(limit_us, parked):
    from nvfp4_training_b200 import _lib as L
    lib = L.load()
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    L.check(lib.nvfp4_selftest_wait_timeout(limit_us, parked, st.data_ptr(), L.stream()), "selftest")
    torch.cuda.synchronize()                       # the kernel ends by itself: the context stays usable
    word = int(st.item())
    assert word & 1, "the limited wait did not report its expiry"
    assert word & 2, "the second warp did not leave through the abort flag"
    waited_us = word >> 8
    # gave up after the limit, and well before the library's default limit of one second
    assert limit_us <= waited_us <= limit_us + 20000, waited_us
    # the context is alive: an ordinary kernel of the library still runs
    from nvfp4_training_b200 import nvq
    assert nvq.amax(torch.full((64,), -3.0, dtype=torch.bfloat16, device="cuda")).item() == 3.0


def test_check_status_reads_both_words():
    from nvfp4_training_b200 import _lib as L
    L.load()
    L.check_status()                               # clean state: no exception
    L.status_word(torch.cuda.current_device()).fill_(12)
    with pytest.raises(L.Nvfp4Error, match="GEMM"):
        L.check_status()
    L.check_status()                               # the word was cleared by the failed check
    out = ctypes.c_int(-1)
    L.check(L.load().nvfp4_quant_tile_status(ctypes.byref(out), 0), "status")
    assert out.value == 0


def test_scheduler_reset_entry_point():
    """`nvfp4_gemm_reset_scheduler` clears the work counters of the CTA-pair GEMM (needed only after an abandoned
    launch): callable at any time between launches, GEMMs before and after it give the same bytes."""
    import torch
    from nvfp4_training_b200 import _lib as L, nvq
    lib = L.load()
    torch.manual_seed(0)
    qa = nvq.quant_rows(torch.randn(512, 2048, device="cuda").bfloat16())
    qb = nvq.quant_rows(torch.randn(768, 2048, device="cuda").bfloat16())
    y0 = nvq.mm(qa, qb)
    torch.cuda.synchronize()
    assert lib.nvfp4_gemm_reset_scheduler() == 0
    y1 = nvq.mm(qa, qb)
    assert torch.equal(y0, y1) and y0.abs().max().item() > 0
    L.check_status()
