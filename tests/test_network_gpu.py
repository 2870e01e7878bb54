"""Whole-network parity: ResNet-50 v1.5 and MobileNetV1 int8 on the GPU against the oracle
forward pass, tensor by tensor, bit for bit."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch

import net_oracle
from helpers import ROOT

pytestmark = pytest.mark.gpu


def nets():
    sys.path.insert(0, os.path.join(ROOT, "paddle-lite_b200"))
    return importlib.import_module("paddle-lite_b200.networks")


@pytest.mark.parametrize("name", ["mobilenet_v1", "resnet50"])
def test_network_bit_exact(plb, ctx, name):
    N = nets()
    spec = N.SPECS[name]()
    qnet = N.build_quantized(spec, seed=7, calib_images=4, device="cuda")
    batch = 2
    rng = np.random.default_rng(99)
    images = rng.standard_normal((batch,) + spec["image"]).astype(np.float32)
    runner = N.Runner(plb, ctx, qnet, batch)
    logits = runner.forward(torch.from_numpy(images).cuda())
    ctx.sync()
    want = net_oracle.forward(qnet, images)
    for key, ref in want.items():
        if key not in runner.buf:
            continue
        got = runner.buf[key].cpu().numpy()
        if got.ndim == 4:
            got = got.transpose(0, 3, 1, 2)[:, :ref.shape[1]]
        assert np.array_equal(got, ref), "tensor %s differs from the oracle (%d of %d elements)" % (
            key, int((got != ref).sum()), ref.size)
    assert np.array_equal(logits.cpu().numpy(), want["logits"])
    assert np.isfinite(want["logits"]).all() and np.abs(want["logits"]).max() > 0


def test_mobilenet_with_fused_depthwise_pairs(plb, ctx, monkeypatch):
    """MobileNetV1 with every qualifying depthwise + 1x1 pair in one launch (blocks 1 - 6): same logits and
    same 1x1 outputs as the oracle, and six launches fewer."""
    N = nets()
    spec = N.SPECS["mobilenet_v1"]()
    qnet = N.build_quantized(spec, seed=7, calib_images=4, device="cuda")
    rng = np.random.default_rng(99)
    images = rng.standard_normal((2,) + spec["image"]).astype(np.float32)
    monkeypatch.setenv("PLB_DWPW", "1")
    runner = N.Runner(plb, ctx, qnet, 2)
    fused = [st for st in runner.steps if st[0] == "dwpw"]
    assert len(fused) == 6
    before = ctx.dwpw_launch_count()
    logits = runner.forward(torch.from_numpy(images).cuda())
    ctx.sync()
    assert ctx.dwpw_launch_count() == before + 6
    want = net_oracle.forward(qnet, images)
    for key, ref in want.items():
        if key not in runner.buf or runner.buf[key].ndim != 4:
            continue
        got = runner.buf[key].cpu().numpy().transpose(0, 3, 1, 2)[:, :ref.shape[1]]
        assert np.array_equal(got, ref), "tensor %s differs from the oracle" % key
    assert np.array_equal(logits.cpu().numpy(), want["logits"])


def test_graph_replay_matches_eager(plb, ctx):
    """The benchmark replays the forward pass as a CUDA graph; the replay must give the same
    logits as the eager enqueue."""
    N = nets()
    spec = N.SPECS["mobilenet_v1"]()
    qnet = N.build_quantized(spec, seed=3, calib_images=2, device="cuda")
    stream = torch.cuda.Stream()
    c2 = plb.Context(0, stream=stream)
    runner = N.Runner(plb, c2, qnet, 4)
    images = torch.randn((4,) + spec["image"], device="cuda")
    with torch.cuda.stream(stream):
        eager = runner.forward(images).clone()
        c2.sync()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            runner.forward(images)
        runner.buf["logits"].zero_()
        g.replay()
        c2.sync()
    assert torch.equal(runner.buf["logits"], eager)


@pytest.mark.parametrize("name,batch", [("resnet50", 128), ("mobilenet_v1", 256)])
def test_benchmark_batch_matches_small_batch(plb, ctx, name, batch):
    """The plan of a layer (tile width, accumulator buffers, resident filter, window mode, strip
    height) depends on the batch.  At the benchmark's batch every tensor of image i must equal the
    same tensor of the two-image run, which the test above ties to the oracle bit for bit."""
    N = nets()
    spec = N.SPECS[name]()
    qnet = N.build_quantized(spec, seed=7, calib_images=4, device="cuda")
    rng = np.random.default_rng(99)
    two = torch.from_numpy(rng.standard_normal((2,) + spec["image"]).astype(np.float32)).cuda()
    small = N.Runner(plb, ctx, qnet, 2)
    small.forward(two)
    ctx.sync()
    big = N.Runner(plb, ctx, qnet, batch)
    big.forward(two.repeat(batch // 2, 1, 1, 1))
    ctx.sync()
    checked = 0
    for key, ref in small.buf.items():
        if key not in big.buf or ref.shape[1:] != big.buf[key].shape[1:]:
            continue
        got = big.buf[key]
        for first in (0, batch - 2):
            assert torch.equal(got[first:first + 2], ref), "tensor %s differs at images %d.." % (key, first)
        checked += 1
    assert checked > 10


@pytest.mark.parametrize("name,batch", [("mobilenet_v1", 40), ("resnet50", 24)])
def test_stem_role_loops_agree(plb, ctx, name, batch, monkeypatch):
    """The stem's window tiles run through short producer / MMA loops; the generic loops
    (PLB_TC_FAST_WINDOW=0) must give the same tensors (several tiles per CTA at this batch)."""
    N = nets()
    spec = N.SPECS[name]()
    qnet = N.build_quantized(spec, seed=5, calib_images=2, device="cuda")
    images = torch.randn((batch,) + spec["image"], device="cuda")
    fast = N.Runner(plb, ctx, qnet, batch)
    fast.forward(images)
    ctx.sync()
    monkeypatch.setenv("PLB_TC_FAST_WINDOW", "0")
    generic = N.Runner(plb, ctx, qnet, batch)
    generic.forward(images)
    ctx.sync()
    for key, ref in generic.buf.items():
        assert torch.equal(fast.buf[key], ref), "tensor %s differs between the role loops" % key
