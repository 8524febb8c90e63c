"""The bounded wait of the cross-GPU rendezvous kernel, on ONE GPU: both ranks' slot arrays live on the local device
and the second rank is played by the test.  Nothing here waits for longer than a few milliseconds: the kernel gives
up after its limit, records TANGO_ETIMEOUT and returns."""
import struct

import pytest
import torch

pytestmark = pytest.mark.gpu

TANGO_ETIMEOUT = -4
LIMIT_NS = 5_000_000       # 5 ms


def _word(round_no: int, value: float) -> int:
    bits = struct.unpack("<I", struct.pack("<f", value))[0]
    w = (round_no << 32) | bits
    return w - (1 << 64) if w >= (1 << 63) else w


def test_rendezvous_wait_expires_reports_and_recovers(cuda):
    from tango_b200._lib import lib
    world = 2
    dev = torch.device("cuda", 0)
    slots = [torch.zeros(2 * world, dtype=torch.int64, device=dev) for _ in range(world)]
    ptrs = torch.tensor([s.data_ptr() for s in slots], dtype=torch.int64, device=dev)
    rnd = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(world)]
    status = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(world)]
    st = torch.cuda.current_stream().cuda_stream

    def call(rank, value):
        v = torch.tensor([value], dtype=torch.float32, device=dev)
        out = torch.full((1,), float("nan"), device=dev)
        rc = lib.tango_peer_sync(ptrs.data_ptr(), rank, world, rnd[rank].data_ptr(), v.data_ptr(), out.data_ptr(),
                                 status[rank].data_ptr(), LIMIT_NS, st)
        assert rc == 0
        torch.cuda.synchronize()
        return float(out)

    # rendezvous 1: rank 1 never arrives -> rank 0 gives up after the limit, says so, and returns its own value
    got = call(0, 3.0)
    assert int(status[0]) == TANGO_ETIMEOUT
    assert got == 3.0
    assert int(rnd[0]) == 1
    # the late rank arrives in rendezvous 1: rank 0's word is there, so it neither waits long nor reports anything
    got = call(1, 7.0)
    assert int(status[1]) == 0 and got == 7.0
    # rendezvous 2: the other rank's word is in place before rank 0 calls (written here as the peer's kernel would) ->
    # the rendezvous completes, the maximum is taken over both ranks, and the status word is left alone
    status[0].zero_()
    for s in slots:
        s[(2 & 1) * world + 1] = _word(2, 11.0)
    got = call(0, 5.0)
    assert int(status[0]) == 0 and got == 11.0 and int(rnd[0]) == 2
    # a word that still carries an older rendezvous number does not take part in the maximum
    status[0].zero_()
    got = call(0, 2.0)            # rendezvous 3, bank 1 holds rank 1's word of rendezvous 1 (7.0): expires, 7.0 must be ignored
    assert int(status[0]) == TANGO_ETIMEOUT and got == 2.0
