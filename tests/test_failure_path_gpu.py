"""The failure path of the tensor-core kernel, exercised without faulting or hanging the GPU.

Every pipeline wait in the kernel is bounded.  A wait that runs out records a code in the ctx status
word, the CTA waits (bounded again) for its own copies in flight, frees its tensor memory and
returns; `plb_ctx_sync` / `plb_copy_d2h` then report PLB_E_DEVICE and the context stays usable.

To make a wait run out, a second build of the library (paddle-lite_b200/build.py build_fault_test():
same sources with -DPLB_TC_FAULT_TEST and a wait limit of a few microseconds) lets CTA 0 drop the
copies of one pipeline stage when PLB_TC_TEST_SKIP_LOAD=1: the stage is neither armed nor fetched, so
the MMA warp's wait for it ends at its limit.  Nothing traps, spins without bound or touches a bad
address.  The library is chosen with PLB200_LIBRARY, hence the child process.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import importlib, os, sys
import numpy as np
import torch
sys.path.insert(0, os.path.join(ROOT, "tests"))
from helpers import O, conv_case
plb = importlib.import_module("paddle-lite_b200")
torch.cuda.set_device(0)
ctx = plb.Context(0)
xq, in_s, wq, ws, bias = conv_case(31, 8, 64, 28, 28, 128, 1)
want = O.conv_int8(xq, wq, ws, in_s, bias, O.ACT_RELU, out_scale=0.05)
x = ctx.nchw_to_nhwc_i8(torch.from_numpy(xq).cuda())
ctx.sync()

def layer():
    return plb.Conv(ctx, wq, ws, in_s, bias, in_hw=(28, 28), act=plb.ACT_RELU, out_scale=0.05)

def check_good(tag):
    y = layer().run_nhwc(x)
    ctx.sync()
    assert np.array_equal(ctx.nhwc_to_nchw(y).cpu().numpy(), want), tag + ": result differs from the oracle"

os.environ["PLB_TC_TEST_SKIP_LOAD"] = "0"
check_good("before the fault")

# 1. a lost stage: the MMA warp's wait runs out, plb_ctx_sync reports it and names the block
os.environ["PLB_TC_TEST_SKIP_LOAD"] = "1"
y = layer().run_nhwc(x)
try:
    ctx.sync()
    raise SystemExit("plb_ctx_sync did not report the lost wait")
except plb.PlbError as e:
    assert e.code == plb.E_DEVICE, e
    assert "block 0" in str(e) and "wait" in str(e), str(e)
ctx.sync()  # the flag was cleared: the ctx is usable again

# 2. the same through the host copy the io_copy kernel uses
y = layer().run_nhwc(x)
host = np.empty(y.numel(), dtype=np.int8)
try:
    ctx.copy_d2h(host, y)
    raise SystemExit("plb_copy_d2h did not report the lost wait")
except plb.PlbError as e:
    assert e.code == plb.E_DEVICE, e

# 3. the next launches on the same ctx are bit-exact again
os.environ["PLB_TC_TEST_SKIP_LOAD"] = "0"
check_good("after the fault")
check_good("after the fault, again")
print("FAILURE_PATH_OK")
'''


def test_lost_pipeline_stage_is_reported_and_the_ctx_survives(plb):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    sys.path.insert(0, os.path.join(ROOT, "paddle-lite_b200"))
    import build as plb_build
    lib = plb_build.build_fault_test()
    env = dict(os.environ, PLB200_LIBRARY=lib,
               PLB_TC_FAST_FLAT="0", PLB_TC_FAST_IM2COL="0")  # the generic producer loop carries the test hook
    code = "ROOT = %r\n" % ROOT + "import sys\nsys.path.insert(0, ROOT)\n" + CHILD
    r = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "FAILURE_PATH_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
