"""A barrier wait that runs out inside the tensor-core step: the kernel returns, the sticky flag
reaches the host, and the context stays usable.

No GPU fault is involved.  KMB_TC_TEST_STALL=1 makes the sample-tile producer of every CTA stop
after its first tile (a copy that never arrives), KMB_TC_TIMEOUT_MS shortens the limit of the
waits to 200 ms; the warps waiting for the second tile give up, every role leaves its loop, the
producers and MMA warps wait for what they still have in flight, tensor memory is released and
the kernel ends.  The switches are read at launch time, so the same child process then runs a
normal step on the same device and checks its labels.
"""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = textwrap.dedent("""
    import os, sys, time
    import numpy as np, torch
    sys.path.insert(0, os.getcwd())
    from sklearn_numba_dpex_b200._cabi import KmbError, check, lib, ptr, stream_ptr
    from sklearn_numba_dpex_b200.kmeans.drivers import LloydState

    d = int(sys.argv[1])
    n, k = 148 * 128 * 3 + 77, 256                # three sample tiles per CTA and a ragged last one
    g = torch.Generator(device="cuda").manual_seed(5)
    X = torch.randn((n, d), device="cuda", generator=g)
    C = X[torch.randperm(n, device="cuda", generator=g)[:k]].clone()

    os.environ["KMB_TC_TEST_STALL"] = "1"
    os.environ["KMB_TC_TIMEOUT_MS"] = "200"
    st = LloydState(X, None, C, "tf32x3")
    assert st.is_tc
    t0 = time.time()
    try:
        st.step()
    except KmbError as exc:
        assert "bounded wait" in str(exc), exc
    else:
        raise SystemExit("the stalled step did not report its wait")
    torch.cuda.synchronize()
    elapsed = time.time() - t0
    assert elapsed < 20.0, elapsed                 # a few 200 ms limits, not the default 2 s ones
    try:
        st.check_device_waits()
    except KmbError:
        pass
    else:
        raise SystemExit("the flag is not sticky")

    # the same context, switches off: a clean workspace and a normal step
    os.environ["KMB_TC_TEST_STALL"] = "0"
    os.environ["KMB_TC_TIMEOUT_MS"] = "0"
    st2 = LloydState(X, None, C, "tf32x3")
    st2.step()
    st2.check_device_waits()
    ref = LloydState(X, None, C, "cuda_core")
    ref.step()
    a, b = st2.labels.cpu().numpy(), ref.labels.cpu().numpy()
    assert (a != b).mean() < 1e-4, (a != b).mean()  # near-ties only
    print("stall-ok %.2f s" % elapsed)
""")


@pytest.mark.parametrize("d,small", [(64, None), (128, None), (16, "3"), (28, "3"), (16, "1"), (16, "ss")],
                         ids=["general_d64", "general_d128", "quads_d16", "quads_d28", "sixteen_d16",
                              "quads_ss_d16"])
def test_wait_that_runs_out_is_reported_and_the_context_survives(d, small):
    env = dict(os.environ)
    if small == "ss":
        env["KMB_TQ_SS"] = "1"
    elif small is not None:
        env["KMB_TC_SMALL"] = small
    proc = subprocess.run([sys.executable, "-c", CHILD, str(d)], cwd=ROOT, env=env,
                          capture_output=True, text=True, timeout=600)
    tail = (proc.stdout + proc.stderr)[-3000:]
    assert proc.returncode == 0, tail
    assert "stall-ok" in proc.stdout, tail
