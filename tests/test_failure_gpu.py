"""Failure path of the device-side bounded waits, without faulting or hanging the GPU: a stream-K launch in which the
programs that hold the tail of a tile's K range never raise their "partial published" flag (a test switch of the library, set on the caller's MatmulConfig).
The tile owners' wait runs out after the configured bound, the kernel records a status code and returns normally, the
host reads the code, and the context stays usable for the next launch."""
import pytest
import torch

import tritonblas_b200 as tb
from tests._util import assert_close_to_oracle, make_operands

pytestmark = pytest.mark.gpu


def test_owner_wait_times_out_cleanly_and_context_survives():
    m, n, k = 128, 256, 8192
    a, b = make_operands(m, n, k, torch.bfloat16, "T", "T", seed=1)
    sel = tb.OrigamiMatmulSelector(m, n, k, torch.bfloat16, torch.bfloat16, torch.bfloat16, torch.device("cuda", 0), streamk=True)
    sel.override(cta_pair=1, block_n=128, sk_grid=4)        # 2 tiles over 4 programs: each tile has one owner, one peer
    cfg = tb.matmul_preamble(sel)
    c = torch.zeros(m, n, dtype=torch.bfloat16, device="cuda")
    assert tb.device_status() == 0
    cfg.debug_flags, cfg.wait_timeout_ms = 4, 150     # peers never publish; waits give up after 150 ms
    try:
        tb.streamk_matmul_lt(a, b, c, sel, cfg, sk_grid=4)
        torch.cuda.synchronize()                # the launch itself completes: waits are bounded
    finally:
        cfg.debug_flags, cfg.wait_timeout_ms = 0, 0
    code = tb.device_status()
    assert code == 105, code                    # stream-K owner timed out waiting for a peer's partial tile
    assert tb.device_status() == 0              # reading clears it
    with pytest.raises(tb.TritonBlasError, match="device-side failure"):
        cfg.debug_flags, cfg.wait_timeout_ms = 4, 150
        try:
            tb.streamk_matmul_lt(a, b, c, sel, cfg, sk_grid=4)
        finally:
            cfg.debug_flags, cfg.wait_timeout_ms = 0, 0
        tb.raise_on_device_failure()
    # the same workspace and context keep working
    tb.streamk_matmul_lt(a, b, c, sel, cfg, sk_grid=4)
    assert_close_to_oracle(c, a, b, what="stream-K after a timed-out launch")
    assert tb.device_status() == 0
