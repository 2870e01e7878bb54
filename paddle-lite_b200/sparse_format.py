"""The weight encoding that `sparse_conv2d` consumes, built with numpy.

`encode(w, hw, semi)` reproduces what the reference's optimiser pass writes into the
NonZeroWeights / OcNonZeros / Diffs tensors and the first_ic / flag_semi attributes
(lite/core/optimizer/mir/sparse_conv_detect_pass.cc:35-301):

  * int8 weights, unstructured (:35-91): values in (output channel, input channel) order,
    cumulative counts per output channel, one diff per value = byte distance to the next
    non-zero's input channel times hw; the last diff of every channel is replaced by the running
    sum of all diffs so far (= where the next channel starts, relative to first_ic); the very
    last diff wraps back to first_ic.
  * fp32 weights, unstructured (:93-194): the same with every channel padded to a multiple of
    four entries (zero weight, zero diff); cumulative counts include the padding of the
    previous channels.
  * semi-structured (:196-301): pairs of output channels share one diff per stored 2x1 block
    and store both weights of the block; an odd last channel is stored one value per block.

It is used to build benchmark and example inputs; a deployment gets these tensors from the
reference's own pass.
"""
import numpy as np


def _running_sum(diffs, cum):
    run, ik = 0, 0
    prev = 0
    for c in cum:
        cnt = int(c) - prev
        prev = int(c)
        for _ in range(cnt):
            run += int(diffs[ik])
            ik += 1
        if ik:
            diffs[ik - 1] = run
    return diffs


def encode(w, hw, semi=False):
    w = np.ascontiguousarray(w)
    m, k = w.shape
    is_i8 = w.dtype == np.int8
    esz = 1 if is_i8 else 4
    if not is_i8:
        w = w.astype(np.float32)
    vals, ics, cum = [], [], []
    if semi:
        pairs = m // 2
        for p in range(pairs):
            cols = np.nonzero((w[2 * p] != 0) | (w[2 * p + 1] != 0))[0]
            for ic in cols:
                vals += [w[2 * p, ic], w[2 * p + 1, ic]]
                ics.append(int(ic))
            cum.append(len(ics))
        if m % 2:
            cols = np.nonzero(w[m - 1])[0]
            for ic in cols:
                vals.append(w[m - 1, ic])
                ics.append(int(ic))
            cum.append(len(ics))
        diffs = np.zeros(max(len(ics), 1), dtype=np.int64)
        for t in range(len(ics) - 1):
            diffs[t] = (ics[t + 1] - ics[t]) * esz * hw
        diffs = _running_sum(diffs, cum)
        first_ic = ics[0] if ics else 0
        if ics:
            diffs[len(ics) - 1] = (first_ic - ics[-1]) * esz * hw
        oc = np.zeros(m, dtype=np.uint32)
        oc[:len(cum)] = cum
        return dict(nonzero_weights=np.array(vals, dtype=w.dtype), oc_nonzeros=oc,
                    diffs=diffs[:len(ics)].astype(np.int32), first_ic=first_ic, flag_semi=1)
    pad4 = not is_i8
    stored_ic, real = [], []   # per stored slot: input channel (or None for padding), is-real flag
    for oc_i in range(m):
        cols = np.nonzero(w[oc_i])[0]
        for ic in cols:
            vals.append(w[oc_i, ic])
            stored_ic.append(int(ic))
            real.append(True)
        end_real = len(vals)
        if pad4:
            while len(vals) % 4:
                vals.append(w.dtype.type(0))
                stored_ic.append(None)
                real.append(False)
        cum.append(end_real)
    real_ics = [ic for ic in stored_ic if ic is not None]
    first_ic = real_ics[0] if real_ics else 0
    raw = []
    for t in range(len(real_ics)):
        nxt = real_ics[t + 1] if t + 1 < len(real_ics) else first_ic
        raw.append((nxt - real_ics[t]) * esz * hw)
    diffs = np.zeros(max(len(vals), 1), dtype=np.int64)
    it = iter(raw)
    for slot, is_real in enumerate(real):
        diffs[slot] = next(it) if is_real else 0
    if is_i8:
        if real_ics:
            wrap = diffs[len(vals) - 1]
            diffs[len(vals) - 1] = 0
            diffs = _running_sum(diffs, cum)
            diffs[len(vals) - 1] = wrap
    else:
        diffs = _running_sum(diffs, cum)
    return dict(nonzero_weights=np.array(vals, dtype=w.dtype), oc_nonzeros=np.array(cum, dtype=np.uint32),
                diffs=diffs[:len(vals)].astype(np.int32), first_ic=first_ic, flag_semi=0, pad4=int(pad4))


def quantize_per_channel(w):
    """Per-output-channel symmetric int8: scale = max|w|/127 (quant_dequant_op_fuser.cc:57-73)."""
    amax = np.maximum(np.abs(w).max(axis=1, keepdims=True), 1e-12)
    scale = (amax / 127.0).astype(np.float32)
    return np.clip(np.rint(w / scale), -127, 127).astype(np.int8), scale.reshape(-1)
