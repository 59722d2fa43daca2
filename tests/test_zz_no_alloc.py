"""The allocation-free resize entry point against the ordinary batch path.

Hosts that cannot let a library allocate device memory while they run (a training job whose allocator owns all of
HBM, a no-allocation-after-start-up service) call dg_resize_device_static with their own input and output buffers;
everything else comes from a fixed array inside the library.  Here the caller's buffers are torch tensors, the call
goes through the C ABI, and the result must equal what the batch entry points produce for the same image, bit for bit
(the tolerance of the other resize tests).  Two calls in a row check that what the first call left in the shared
array does not leak into the second.  The file sorts last so that a failure here cannot hide another test.
"""
import numpy as np
import pytest

import datago_b200 as dg

pytestmark = pytest.mark.gpu

CFG = dict(crop_and_resize=True, default_image_size=512, downsampling_ratio=16, min_aspect_ratio=0.5, max_aspect_ratio=2.0)


def _static_vs_batch(ctx, img, forced_key=None):
    import torch
    h, w = img.shape[:2]
    c = 1 if img.ndim == 2 else 3
    plan = ctx.plan_geometry(w, h, c, forced_key)
    src = torch.from_numpy(img).cuda()
    dst = torch.zeros((plan.target_h, plan.target_w) if c == 1 else (plan.target_h, plan.target_w, 3), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    got_plan = ctx.resize_device_static(src.data_ptr(), w, h, c, dst.data_ptr(), forced_key)
    (status, want, res), = ctx.process([img], [forced_key])
    assert status == 0
    assert got_plan.as_tuple() == res.plan.as_tuple()
    assert np.array_equal(dst.cpu().numpy(), want)


def test_two_calls_in_a_row_match_the_batch_path():
    ctx = dg.Context(0, CFG)
    rng = np.random.default_rng(41)
    first = rng.integers(0, 256, (900, 1400, 3), dtype=np.uint8)     # downscale, side crop
    second = rng.integers(0, 256, (700, 333), dtype=np.uint8)        # grayscale, upscale on one axis, other passes
    _static_vs_batch(ctx, first)
    _static_vs_batch(ctx, second)
    _static_vs_batch(ctx, first, "1.000")                            # forced bucket, and the array is dirty by now


def test_source_that_ends_where_its_allocation_could_end():
    # The entry point must not load a byte outside [src, src + w * h * c): the caller's image may end exactly where a
    # mapping ends.  Here the image is an interior slice of a larger tensor (so nothing can leave the allocation
    # whatever the kernel does), at start offsets of every residue modulo 4 and with sizes whose filter windows are not
    # multiples of four taps; the bytes around it are sentinels that would change the result if they leaked into it.
    import torch
    ctx = dg.Context(0, CFG)
    rng = np.random.default_rng(43)
    for (h, w, c), lead in (((301, 1234, 3), 1), ((777, 509, 1), 3), ((640, 1001, 3), 2), ((333, 700, 1), 5), ((512, 515, 3), 7)):
        img = rng.integers(0, 256, (h, w, c), dtype=np.uint8) if c == 3 else rng.integers(0, 256, (h, w), dtype=np.uint8)
        n = h * w * c
        (status, want, res), = ctx.process([img])
        assert status == 0
        for sentinel in (0, 255):
            big = torch.full((lead + n + 64,), sentinel, dtype=torch.uint8, device="cuda")
            big[lead:lead + n] = torch.from_numpy(img.reshape(-1)).cuda()
            dst = torch.zeros(want.shape, dtype=torch.uint8, device="cuda")
            torch.cuda.synchronize()
            ctx.resize_device_static(big.data_ptr() + lead, w, h, c, dst.data_ptr())
            assert np.array_equal(dst.cpu().numpy(), want), (h, w, c, lead, sentinel)


def test_identity_and_copy_only_plans():
    ctx = dg.Context(0, CFG)
    rng = np.random.default_rng(42)
    _static_vs_batch(ctx, rng.integers(0, 256, (512, 512, 3), dtype=np.uint8))          # already the bucket size
    _static_vs_batch(ctx, rng.integers(0, 256, (512, 520, 3), dtype=np.uint8), "1.000")  # same scale, integral crop


def test_oversized_input_is_refused_without_launching():
    import torch
    ctx = dg.Context(0, CFG)
    # a tall, thin image forced into the widest bucket: the resized image is 720 x 115200, far beyond the 32 MiB array
    src = torch.zeros((16000, 100, 3), dtype=torch.uint8, device="cuda")
    dst = torch.full((352, 720, 3), 7, dtype=torch.uint8, device="cuda")
    with pytest.raises(dg.DatagoB200Error) as e:
        ctx.resize_device_static(src.data_ptr(), 100, 16000, 3, dst.data_ptr(), "2.045")
    assert e.value.code == 11 and "static scratch" in str(e.value)
    assert int(dst.min()) == 7 and int(dst.max()) == 7
