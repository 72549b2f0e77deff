"""Helpers shared by the GPU parity tests."""

import torch


def cu(t):
    return None if t is None else t.cuda().contiguous()


def bits(t):
    """Bit pattern view for exact comparison of 16-bit float tensors."""
    if t.dtype in (torch.float16, torch.bfloat16):
        return t.contiguous().view(torch.int16)
    if t.dtype == torch.float32:
        return t.contiguous().view(torch.int32)
    return t


def assert_bit_equal(got, want, what=""):
    got = got.cpu()
    assert got.shape == want.shape, (what, got.shape, want.shape)
    if not torch.equal(bits(got), bits(want)):
        diff = (bits(got) != bits(want))
        n = int(diff.sum())
        idx = diff.nonzero()[:5].tolist()
        raise AssertionError("%s: %d of %d elements differ, first at %s: got %s want %s" % (
            what, n, diff.numel(), idx, [got[tuple(i)].item() for i in idx], [want[tuple(i)].item() for i in idx]))


def mismatch_fraction(got, want):
    return float((got.cpu() != want).float().mean())


def rel_err(got, want):
    g = got.cpu().double()
    w = want.double()
    return float((g - w).norm() / w.norm().clamp_min(1e-30))


def check_status():
    from lyradiff_b200 import ops
    st, detail = ops.last_status()
    assert st == 0, "device status %d detail 0x%x" % (st, detail)
