"""The no-allocation dispatch entry point (moe_b200_dispatch_static) against the regular one.

Collected last on purpose (file name), so a run that stops at the first failure has already been
through every other test. The entry point exists for hosts that must not allocate device memory at
call time (a frozen memory plan, or a foreign-function caller without a device allocator): its
scratch is a fixed array inside the library, shared by all calls on a device. The test therefore
makes two calls in a row with different inputs and checks that the second is not polluted by what
the first left in that array. Calls go straight through the C ABI; the only buffers are the
inputs and outputs the caller owns."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _static_dispatch(lib, idx, n_experts, status):
    from nanospeaker_b200 import kernels
    flat = idx.reshape(-1).contiguous()
    m = flat.numel()
    cap = kernels.l_cap(m, n_experts)
    dev, i32 = flat.device, torch.int32
    outs = [torch.full((cap,), -7, dtype=i32, device=dev),
            torch.full((cap // 128,), -7, dtype=i32, device=dev),
            torch.full((n_experts + 1,), -7, dtype=i32, device=dev),
            torch.full((n_experts,), -7, dtype=i32, device=dev),
            torch.full((1,), -7, dtype=i32, device=dev),
            torch.full((m,), -7, dtype=i32, device=dev)]
    rc = lib.moe_b200_dispatch_static(
        flat.data_ptr(), m, n_experts, *[o.data_ptr() for o in outs], status.data_ptr(),
        torch.cuda.current_stream().cuda_stream)
    return rc, outs


def test_static_dispatch_matches_regular_dispatch_twice_in_a_row():
    from nanospeaker_b200 import _lib, kernels
    lib = _lib.load()
    status = kernels.status_word("cuda")
    torch.manual_seed(7)
    cases = [
        (torch.randn(16384, 76, device="cuda") + 1.5 * torch.randn(76, device="cuda"), 76, 6),
        (torch.randn(5000, 8, device="cuda"), 8, 2),     # fewer experts: stale entries in reach
    ]
    for logits, n_experts, k in cases:
        idx = logits.topk(k, dim=-1).indices
        rc, got = _static_dispatch(lib, idx, n_experts, status)
        assert rc == 0, _lib.error_string(rc)
        want = kernels.dispatch(idx, n_experts)
        torch.cuda.synchronize()
        live_tiles = int(want[4]) // 128
        names = ["sorted_ids", "expert_ids", "pad_offsets", "counts", "n_post_pad", "inv_ids"]
        for name, a, b in zip(names, got, want):
            if name == "expert_ids":
                a, b = a[:live_tiles], b[:live_tiles]
            assert torch.equal(a, b), name               # integer plan: bit-exact
    kernels.check_status("cuda")


def test_static_dispatch_rejects_sizes_beyond_its_scratch():
    from nanospeaker_b200 import _lib
    lib = _lib.load()
    # the array holds 128 blocks x 256 experts, the most the dispatch ever uses, so the limit is
    # the dispatch's own cap on the pair count
    assert lib.moe_b200_dispatch_static_max_pairs(76) == 1 << 30
    assert lib.moe_b200_dispatch_static_max_pairs(256) == 1 << 30
    assert lib.moe_b200_dispatch_static_max_pairs(0) == 0
    assert lib.moe_b200_dispatch_scratch_bytes(1 << 30, 256) <= 128 * 1024
    too_many = lib.moe_b200_dispatch_static_max_pairs(256) + 1
    buf = torch.zeros(16, dtype=torch.int32, device="cuda")
    p = buf.data_ptr()
    rc = lib.moe_b200_dispatch_static(p, too_many, 256, p, p, p, p, p, p, p, 0)
    assert rc == -8 and "scratch" in _lib.error_string(rc)
