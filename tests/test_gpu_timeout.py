"""A bounded device wait that runs out: the kernel returns, b200q_sync reports Timeout, the context
stays usable.  The wait is made to run out on the host's terms (a peer that never posts: the second
"rank" is a context that simply does not call), with the wait limit set to 50 ms; nothing faults,
traps or hangs.  One GPU: the two contexts live on the same device and only one of them launches."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import magnitude_b200 as mb  # noqa: E402
from magnitude_b200 import _binding as B  # noqa: E402
from magnitude_b200 import ggml_quant as gq  # noqa: E402


def test_peer_exchange_times_out_and_the_context_survives(orc):
    a, b = mb.Backend(0), mb.Backend(0)
    try:
        bufs = [a.peer_buffer(), b.peer_buffer()]
        a.peer_attach_buffers(0, 2, bufs)
        b.peer_attach_buffers(1, 2, bufs)
        a.set_option(B.OPT_WAIT_LIMIT_MS, 50)
        y = torch.ones(4096, device="cuda")
        a.allreduce(y)                                   # rank 1 never posts its share
        with pytest.raises(mb.B200QError) as e:
            a.sync()
        assert e.value.status == B.ERR_TIMEOUT
        # the context is not poisoned: an ordinary product still runs and is right
        n, k = 64, 1024
        packed = gq.synth_weights(mb.TYPE_Q4_K, n, k, 1)
        w = a.upload(mb.TYPE_Q4_K, packed, n, k)
        x = torch.randn(1, k, device="cuda").to(torch.bfloat16)
        out = a.project(w, x)
        a.sync()
        ref = orc.matmul_exact(mb.TYPE_Q4_K, packed, n, k, x.float().cpu().numpy())
        assert orc.within_tolerance(out.cpu().numpy(), ref, 1e-3)[0]
        # the ranks' call counters no longer agree: further exchanges are refused until both re-attach
        with pytest.raises(mb.B200QError) as e:
            a.allreduce(y)
        assert e.value.status == B.ERR_STOPPED
        a.peer_detach()
        b.peer_detach()
        a.peer_attach_buffers(0, 1, [a.peer_buffer()])   # a world of one: the sum is the input
        a.allreduce(y)
        a.sync()
        a.peer_detach()
        w.close()
    finally:
        a.set_option(B.OPT_WAIT_LIMIT_MS, 2000)
        a.close()
        b.close()


def test_option_ranges(backend):
    for opt, bad in ((B.OPT_WAIT_LIMIT_MS, 0), (B.OPT_WAIT_LIMIT_MS, 10**7), (B.OPT_TP_INIT_TIMEOUT_MS, 0)):
        with pytest.raises(mb.B200QError):
            backend.set_option(opt, bad)
    backend.set_option(B.OPT_TP_INIT_TIMEOUT_MS, 30000)
