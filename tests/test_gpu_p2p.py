"""Device-side messaging primitives of the expert-parallel decode protocol (the launchers of dsv41/cukern.py:348-434), exercised on one
GPU: destinations and flags are local buffers, every signal precedes its wait on the same stream, and the bounded wait is shown to give
up cleanly (error status, no hang, stream usable) on a flag that nothing sets."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ptrs(tensors, dev):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=dev)


def test_copy_signal_wait_multicast(mods, dev):
    ck = mods.cukern
    src = torch.randn(3, 1024, device=dev)
    dst = torch.zeros(4, 1024, device=dev)
    ck.p2p_copy(dst, src, dev)
    seq = torch.zeros(1, dtype=torch.int32, device=dev)
    ck.p2p_seq_bump(seq, dev)
    ck.p2p_seq_bump(seq, dev)
    flags = torch.zeros(5, dtype=torch.int32, device=dev)
    ck.p2p_signal(_ptrs([flags[1:2], flags[3:4]], dev), seq, dev)
    mask = torch.tensor([0, 1, 0, 1, 0], dtype=torch.int32, device=dev)
    ck.p2p_wait_masked(flags, seq, mask, dev)          # the two signalled flags only
    ck.p2p_wait(flags[1:2], seq, dev)
    inbox = [torch.zeros(2048, device=dev) for _ in range(3)]
    in_flags = torch.zeros(3, dtype=torch.int32, device=dev)
    payload = torch.randn(2048, device=dev)
    ck.p2p_multicast(_ptrs(inbox, dev), payload, _ptrs([in_flags[i:i + 1] for i in range(3)], dev), seq, dev)
    ck.p2p_wait(in_flags, seq, dev)
    stamp = torch.zeros(1, dtype=torch.int64, device=dev)
    ck.p2p_stamp(stamp, dev)
    far = torch.zeros(1024, device=dev)
    ck.memcpy_async(far, src[1], dev)
    torch.cuda.synchronize()
    assert torch.equal(dst[:3], src) and dst[3].abs().sum() == 0
    assert seq.item() == 2 and flags.tolist() == [0, 2, 0, 2, 0] and in_flags.tolist() == [2, 2, 2]
    assert all(torch.equal(b, payload) for b in inbox) and torch.equal(far, src[1]) and stamp.item() > 0
    assert ck.device_error(dev) == 0
    # second use of the self-resetting counter
    ck.p2p_seq_bump(seq, dev)
    ck.p2p_multicast(_ptrs(inbox, dev), payload * 2, _ptrs([in_flags[i:i + 1] for i in range(3)], dev), seq, dev)
    ck.p2p_wait(in_flags, seq, dev)
    torch.cuda.synchronize()
    assert in_flags.tolist() == [3, 3, 3] and torch.equal(inbox[2], payload * 2) and ck.device_error(dev) == 0


def test_copy_row_into_per_sequence_inboxes(mods, dev):
    S, rows, D, B = 3, 5, 64, 4
    base = torch.zeros(S, rows, D, device=dev, dtype=torch.bfloat16)
    src = torch.randn(B, 1, D, device=dev).to(torch.bfloat16)
    row_idx = torch.tensor([4, 0, 2, 2], dtype=torch.int64, device=dev)
    seq = torch.tensor([0, 2, 1, 2], dtype=torch.int64, device=dev)
    mods.cukern.p2p_copy_row(base, row_idx, src, dev, seq)
    torch.cuda.synchronize()
    want = torch.zeros_like(base)
    for b in range(B):
        want[seq[b], row_idx[b]] = src[b, 0]
    assert torch.equal(base, want)


def test_wait_gives_up_after_its_limit(mods, dev):
    """A flag that nothing sets: the wait returns when its limit (2 ms here) has run out and leaves code 3001 (3002 for the masked
    form) in the device error word; the stream keeps working and the next read of the word is clean."""
    ck = mods.cukern
    flags = torch.zeros(2, dtype=torch.int32, device=dev)
    seq = torch.ones(1, dtype=torch.int32, device=dev)
    ck.set_wait_limit_ns(2_000_000)
    try:
        ck.p2p_wait(flags, seq, dev)
        after = torch.full((4,), 7.0, device=dev) * 2        # work queued behind the wait still runs
        assert ck.device_error(dev) == 3001
        assert after.tolist() == [14.0] * 4
        ck.p2p_wait_masked(flags, seq, torch.tensor([0, 1], dtype=torch.int32, device=dev), dev)
        assert ck.device_error(dev) == 3002
        ck.p2p_wait_masked(flags, seq, torch.zeros(2, dtype=torch.int32, device=dev), dev)   # nothing to wait for
        assert ck.device_error(dev) == 0
    finally:
        ck.set_wait_limit_ns(0)
