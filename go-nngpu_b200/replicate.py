"""Replication of B for the row-sharded product: host-side bookkeeping.

Every rank multiplies its own rows of A by the whole of B, so B has to reach
every GPU.  `Replicator` owns a symmetric buffer (the same allocation on every
GPU of the group, bound to an NVSwitch multicast address) with two slots for B
and the control words of `gonngpu_replicate_send` / `gonngpu_replicate_wait`,
and issues those two calls with the right slot, epoch and acknowledgement
numbers:

    epoch e (1, 2, ...) uses slot e % 2
    owner:      send(slot, e, ack_needed = e - 2)   every rank is done with epoch e - 2,
                                                    the last one that used this slot
    every rank: wait(slot, e, ack_value  = e - 1)   my products up to epoch e - 1 are
                                                    complete (they precede this call on
                                                    the stream); then hold until e arrived

The allocation, the exchange of memory handles between the processes and the
multicast binding come from torch's symmetric-memory allocator
(`open_symmetric`); a caller with its own allocator passes the three addresses
to `Replicator` directly.
"""


class Replicator:
    def __init__(self, binding, world, rank, owner, bases_dev, multicast_ptr, slot_bytes, ctrl_offset,
                 ctas=0, data_offset=0, send_stream=None):
        """`data_offset`: where this channel's two slots begin inside the symmetric buffer (several
        channels, one per column slab of B, share one buffer; each has its own 128 bytes of
        control words at `ctrl_offset`).  `send_stream`: cudaStream_t (int) the owner's pushes are
        enqueued on, None = the library's stream."""
        if slot_bytes % 16 or ctrl_offset % 16 or data_offset % 16 or \
                data_offset <= ctrl_offset < data_offset + 2 * slot_bytes:
            raise ValueError("slots are multiples of 16 bytes and the control words lie outside them")
        self.g, self.world, self.rank, self.owner = binding, world, rank, owner
        self.bases, self.mc = bases_dev, multicast_ptr
        self.slot_bytes, self.ctrl, self.ctas = slot_bytes, ctrl_offset, ctas
        self.data_offset, self.send_stream = data_offset, send_stream
        self.epoch = 0

    def slot_offset(self, slot):
        """Byte offset of `slot` inside every rank's symmetric buffer."""
        return self.data_offset + slot * self.slot_bytes

    @property
    def slot(self):
        """Slot that holds the most recent epoch."""
        return self.epoch % 2

    def replicate(self, src_ptr=None):
        """One replication: the owner pushes the bytes at `src_ptr`; every rank (the owner too)
        then holds the library's stream until they have arrived.  Returns the slot the following
        product reads."""
        slot = self.send(src_ptr)
        self.wait()
        return slot

    def wait(self):
        """Second half of `replicate`: acknowledge the previous epoch, wait for the current one."""
        e = self.epoch
        self.g.replicate_wait(self.bases, self.world, self.owner, self.rank, self.ctrl, e % 2, e, e - 1)
        return e % 2

    def send(self, src_ptr=None):
        """First half of `replicate`: opens the next epoch; on the owner, enqueues the push."""
        self.epoch += 1
        e, slot = self.epoch, self.epoch % 2
        if self.rank == self.owner:
            if src_ptr is None:
                self.epoch -= 1
                raise ValueError("the owner passes the source address")
            self.g.replicate_send(src_ptr, self.mc + self.slot_offset(slot), self.slot_bytes, self.bases,
                                  self.world, self.rank, self.ctrl, slot, e, max(e - 2, 0), self.ctas,
                                  self.send_stream)
        return slot


class ShardedProduct:
    """The row-sharded product whose kernel replicates B itself (`gonngpu_gemm_f16_sharded`):
    keeps the epoch, which every rank advances by one per step, and the addresses of the
    symmetric buffer (two slots of B at offset 0, the control words behind them)."""

    def __init__(self, binding, world, rank, owner, local_base, bases_dev, multicast_base, k, n,
                 first_group=0):
        if n % 8:
            raise ValueError("B needs a multiple of 8 columns")
        self.g, self.world, self.rank, self.owner = binding, world, rank, owner
        self.local_base, self.bases, self.mc = local_base, bases_dev, multicast_base
        self.k, self.n, self.first_group = k, n, first_group
        self.slot_bytes = 2 * k * n
        self.ctrl = 2 * self.slot_bytes
        self.epoch = 0

    @property
    def slot(self):
        """Slot that holds the most recent epoch's B."""
        return self.epoch % 2

    def slot_offset(self, slot):
        return slot * self.slot_bytes

    def step(self, a_ptr, rows, a_pitch, c_ptr, ldc, b_src_ptr=None):
        """Enqueues this rank's product of the next epoch; the owner passes where B lies."""
        if self.rank == self.owner and not b_src_ptr:
            raise ValueError("the owner passes the source address")
        self.epoch += 1
        self.g.gemm_f16_sharded(a_ptr, (rows, self.k), a_pitch, b_src_ptr if self.rank == self.owner else None,
                                self.n, self.local_base, self.bases, self.mc, self.world, self.owner,
                                self.rank, 0, self.ctrl, self.epoch, c_ptr, ldc, self.first_group)
        return self.epoch % 2


def open_symmetric(torch, dist, dev, slot_bytes, require_multicast=True):
    """Allocates the symmetric buffer (two slots + one 4 KiB page of control words, zeroed) with
    torch's symmetric-memory allocator and returns (buffer, handle, ctrl_offset).  Raises when the
    group has no multicast address (no NVSwitch, or the driver refuses the binding), unless
    `require_multicast` is False (the handle's multicast_ptr is then 0)."""
    import torch.distributed._symmetric_memory as symm
    buf = symm.empty(2 * slot_bytes + 4096, dtype=torch.uint8, device=dev)
    hdl = symm.rendezvous(buf, dist.group.WORLD)
    if require_multicast and not int(hdl.multicast_ptr):
        raise RuntimeError("no multicast address for the group")
    buf.zero_()
    return buf, hdl, 2 * slot_bytes
