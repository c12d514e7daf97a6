"""The fused row-parallel decode kernel on ONE GPU: the other ranks are emulated by writing their
packets into this rank's receive buffer, or by leaving them out.

* A packet that never arrives: the wait limit is set to a few milliseconds, nobody plays rank 1, and
  the kernel must come back with status 100 + 1, leave the context usable and advance its sequence
  number (no fault, no trap, no unbounded wait: the wait gives up and the kernel returns).
* Packets that are there: the sum over ranks is taken in rank order, bit for bit, for worlds of 2
  and 4 and any position of this rank."""

import ctypes

import numpy as np
import pytest
import torch

import oracle
import mixfp4_b200 as mx
from mixfp4_b200 import _native as nat, synth

pytestmark = pytest.mark.gpu


class _DeviceBytes:
    """A device pointer as an object torch.as_tensor can view (CUDA array interface)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class LocalComm:
    """A communicator of `world` ranks whose peers are plain buffers of this process."""

    def __init__(self, rank: int, world: int, slots: int):
        self.lib = nat.lib()
        self.rank, self.world, self.slots = rank, world, slots
        self.handle = ctypes.c_void_p()
        nat.check("mixfp4_comm_create", self.lib.mixfp4_comm_create(rank, world, slots, ctypes.byref(self.handle)))
        nbytes = self.lib.mixfp4_comm_buffer_bytes(world, slots)
        self.outboxes = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]   # what we send
        ptrs = (ctypes.c_void_p * world)(*[t.data_ptr() for t in self.outboxes])
        nat.check("mixfp4_comm_open_local", self.lib.mixfp4_comm_open_local(self.handle, ptrs))
        own = ctypes.c_void_p()
        nat.check("mixfp4_comm_buffer", self.lib.mixfp4_comm_buffer(self.handle, ctypes.byref(own)))
        self.inbox = torch.as_tensor(_DeviceBytes(own.value, nbytes), device="cuda").view(torch.int32).reshape(-1, 2)
        self.status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def deliver(self, seq: int, src: int, values: torch.Tensor):
        """Write rank src's packets of launch `seq` into this rank's receive buffer."""
        count = values.numel()
        packets = torch.empty((count, 2), dtype=torch.int32, device="cuda")
        packets[:, 0] = values.reshape(-1).contiguous().view(torch.int32)
        packets[:, 1] = seq + 1
        first = ((seq & 1) * self.world + src) * self.slots
        self.inbox[first:first + count] = packets
        torch.cuda.synchronize()

    def launch(self, x, packed, out_dtype=torch.float32):
        m = x.shape[0]
        y = torch.empty((m, packed.n), dtype=out_dtype, device="cuda")
        self.status.zero_()
        st = self.lib.mixfp4_gemv_allreduce(
            self.handle, x.data_ptr(), m, x.stride(0), packed.codes.data_ptr(), nat.ptr(packed.scales),
            packed.global_scale.data_ptr(), nat.ptr(packed.lut), packed.n, packed.k, packed.layout_code, y.data_ptr(),
            nat.DTYPE_CODE[out_dtype], y.stride(0), self.status.data_ptr(), nat.gemv_flags(False, packed.lut),
            nat.stream_ptr(x.device))
        nat.check("mixfp4_gemv_allreduce", st)
        torch.cuda.synchronize()
        return y

    def close(self):
        self.lib.mixfp4_comm_destroy(self.handle)


@pytest.mark.parametrize("layout", ["stream", "kernel"])
def test_a_missing_rank_costs_the_wait_limit_and_a_status_not_a_hang(layout):
    n, k, m = 64, 512, 2
    w = synth.student_t_weight(n, k, 1)
    packed = mx.quantize_packed(w.cuda())[0]
    packed = packed.to_stream_layout() if layout == "stream" else packed.to_kernel_layout()
    x = synth.activations(m, k, 2).cuda()
    own = mx.mixfp4_linear(x, packed, out_dtype=torch.float32)
    comm = LocalComm(rank=0, world=2, slots=m * n)
    lib = nat.lib()
    assert lib.mixfp4_set_wait_limit_ns(5_000_000) == 0           # 5 ms
    try:
        comm.launch(x, packed)                                    # launch 0: rank 1 never sends
        assert int(comm.status.item()) == 101
        value = ctypes.c_int(0)
        rc = lib.mixfp4_check_status(comm.status.data_ptr(), ctypes.byref(value), nat.stream_ptr(x.device))
        assert rc == nat.E_DEVICE_WAIT and value.value == 101
        # what this rank sent to rank 1 is its own partial sums, tagged with launch 0
        sent = comm.outboxes[1].view(torch.int32).reshape(-1, 2)[: m * n]
        assert torch.equal(sent[:, 0].view(torch.float32).reshape(m, n), own) and bool((sent[:, 1] == 1).all())
        # the context is usable and the sequence number advanced: launch 1 finds rank 1's packets
        assert torch.equal(mx.mixfp4_linear(x, packed, out_dtype=torch.float32), own)
        other = torch.full((m, n), 0.75, device="cuda")
        comm.deliver(1, 1, other)
        y = comm.launch(x, packed)
        assert int(comm.status.item()) == 0
        assert torch.equal(y, own + other)
    finally:
        assert lib.mixfp4_set_wait_limit_ns(2_000_000_000) == 0
        comm.close()


@pytest.mark.parametrize("world,rank", [(2, 1), (4, 0), (4, 2), (8, 5)])
@pytest.mark.parametrize("n,k,m", [(272, 1152, 1), (4096, 512, 8), (50, 70, 3)])
def test_partial_sums_are_added_in_rank_order(world, rank, n, k, m):
    w = synth.student_t_weight(n, k, n + k)
    packed = mx.quantize_packed(w.cuda())[0].to_stream_layout()
    x = synth.activations(m, k, 3).cuda()
    own = mx.mixfp4_linear(x, packed, out_dtype=torch.float32)
    ref = oracle.quantize(w.float().numpy())
    ystar = oracle.linear(x.float().cpu().numpy(), oracle.bf16_bits_to_f32(oracle.dequant(ref, "bf16")))
    assert oracle.relative_l2(own.cpu().numpy(), ystar) <= 1e-3
    comm = LocalComm(rank, world, m * n)
    try:
        for seq in range(3):                                       # three launches: both parities, the sequence word
            parts = [own if r == rank else torch.randn((m, n), generator=torch.Generator(device="cuda").manual_seed(10 * seq + r),
                                                       device="cuda") for r in range(world)]
            for r in range(world):
                if r != rank:
                    comm.deliver(seq, r, parts[r])
            want = parts[0].clone()
            for r in range(1, world):
                want = want + parts[r]                             # fp32, rank order
            y = comm.launch(x, packed)
            assert int(comm.status.item()) == 0
            assert torch.equal(y, want)
    finally:
        comm.close()
