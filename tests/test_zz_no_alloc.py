"""The log-mel entry point that carries its own scratch (wdz_logmel_static).

It exists for hosts that cannot give the engine a workspace - a serving
process that has already handed all GPU memory to its own pool, or a loop that
cannot afford the device-wide stall of an allocation - so it must give the
same spectrogram as wdz_logmel while allocating nothing itself.  Both run the
same kernels, so the results are compared bit for bit, on two calls in a row
(the built-in array keeps the previous call's contents and must not leak them
into the next).  Collected last on purpose: a failure here stops nothing else.
"""
import numpy as np
import pytest
import torch

from whisperdrz_b200 import synth
from whisperdrz_b200.dims import ModelDimensions
from whisperdrz_b200.weights import init_state_dict

pytestmark = pytest.mark.gpu


def test_static_scratch_logmel_matches_workspace_logmel_twice():
    from whisperdrz_b200.capi import WdzError
    from whisperdrz_b200.engine import Engine
    dims = ModelDimensions.from_name("test-tiny")
    e = Engine(dims, init_state_dict(dims, 0), dtype=torch.float32, n_slots=2, max_clips=4)
    try:
        # first call: three ragged clips, loud; second call: two quiet clips with a window offset -
        # a stale per-clip maximum from the first call would change the floor of the second
        calls = [
            ([480000, 200000, 16000], [40, 41, 42], 1.0, None),
            ([480000, 333333], [43, 44], 0.01, [100, 7]),
        ]
        for lens, seeds, gain, offs in calls:
            buf = torch.zeros(len(lens), 480000)
            for i, (n, sd) in enumerate(zip(lens, seeds)):
                buf[i, :n] = torch.from_numpy(synth.clip(sd, n / 16000)) * gain
            buf = buf.cuda()
            want = e.logmel(buf, n_samples=lens, frame_offset=offs)
            got = e.logmel_static(buf, n_samples=lens, frame_offset=offs)
            torch.cuda.synchronize()
            assert torch.equal(got, want)
            assert np.isfinite(got.cpu().numpy()).all()
        # beyond the stated maximum the call is refused with a clear error, not truncated
        with pytest.raises(WdzError) as err:
            e.logmel_static(torch.zeros(5, 480000).cuda())
        assert "at most 4" in str(err.value)
    finally:
        e.close()


def test_static_scratch_logmel_needs_no_workspace():
    """An engine that was never lent a workspace: the entry point with built-in scratch still works (and gives
    the spectrogram of an ordinary engine), the workspace-based one reports that it has no memory to work in."""
    from whisperdrz_b200.capi import WdzError
    from whisperdrz_b200.engine import Engine
    dims = ModelDimensions.from_name("test-tiny")
    sd = init_state_dict(dims, 0)
    bare = Engine(dims, sd, dtype=torch.float32, n_slots=2, max_clips=4, lend_workspace=False)
    full = Engine(dims, sd, dtype=torch.float32, n_slots=2, max_clips=4)
    try:
        buf = torch.from_numpy(synth.clips([50, 51])).cuda()
        for _ in range(2):
            got = bare.logmel_static(buf)
            torch.cuda.synchronize()
            assert torch.equal(got, full.logmel(buf))
        with pytest.raises(WdzError) as err:
            bare.logmel(buf)
        assert "WDZ_ENOMEM" in str(err.value)
    finally:
        bare.close()
        full.close()
