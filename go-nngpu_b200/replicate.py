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
                 ctas=0):
        if slot_bytes % 16 or ctrl_offset % 16 or ctrl_offset < 2 * slot_bytes:
            raise ValueError("slots are multiples of 16 bytes and the control words lie behind them")
        self.g, self.world, self.rank, self.owner = binding, world, rank, owner
        self.bases, self.mc = bases_dev, multicast_ptr
        self.slot_bytes, self.ctrl, self.ctas = slot_bytes, ctrl_offset, ctas
        self.epoch = 0

    @property
    def slot(self):
        """Slot that holds the most recent epoch."""
        return self.epoch % 2

    def replicate(self, src_ptr=None):
        """One replication, enqueued on the library's stream: the owner pushes the bytes at
        `src_ptr`; every rank (the owner too) then holds its stream until they have arrived.
        Returns the slot the following product reads."""
        self.epoch += 1
        e, slot = self.epoch, self.epoch % 2
        if self.rank == self.owner:
            if src_ptr is None:
                raise ValueError("the owner passes the source address")
            self.g.replicate_send(src_ptr, self.mc + slot * self.slot_bytes, self.slot_bytes, self.bases,
                                  self.world, self.rank, self.ctrl, slot, e, max(e - 2, 0), self.ctas)
        self.g.replicate_wait(self.bases, self.world, self.owner, self.rank, self.ctrl, slot, e, e - 1)
        return slot


def open_symmetric(torch, dist, dev, slot_bytes):
    """Allocates the symmetric buffer (two slots + one 4 KiB page of control words, zeroed) with
    torch's symmetric-memory allocator and returns (buffer, handle, ctrl_offset).  Raises when the
    group has no multicast address (no NVSwitch, or the driver refuses the binding)."""
    import torch.distributed._symmetric_memory as symm
    buf = symm.empty(2 * slot_bytes + 4096, dtype=torch.uint8, device=dev)
    hdl = symm.rendezvous(buf, dist.group.WORLD)
    if not int(hdl.multicast_ptr):
        raise RuntimeError("no multicast address for the group")
    buf.zero_()
    return buf, hdl, 2 * slot_bytes
