"""One long context split over the GPUs of a box by contiguous key ranges: the host side of the KV-split decode
(ns_b200_kvsplit_decode / ns_b200_kvsplit_combine in include/ns_attn.h).

The reference has nothing like it - it keeps a context on one GPU and moves activations between GPUs through host memory
(kernels/ns/ns.cpp:244-250) - so this follows the benchmark's plan instead: rank r owns keys [r*kv/N, (r+1)*kv/N), every
rank computes its partial (O, m, l), pushes it into every rank's mailbox over NVLink, and merges what arrives in its own.
One process per GPU; torch.distributed carries only the set-up (the 64-byte IPC handles of the mailboxes).
"""
import ctypes as C

import numpy as np

from .core import DevBuf, check


def key_ranges(kv, nranks, multiple=64):
    """[(base, count)] per rank: contiguous, covering 0..kv, every boundary a multiple of `multiple` keys (the last
    rank takes the remainder). Ranks past the end of a short context get (kv, 0)."""
    per = -(-kv // nranks)
    per = -(-per // multiple) * multiple
    out = []
    for r in range(nranks):
        b = min(kv, r * per)
        e = min(kv, (r + 1) * per)
        out.append((b, e - b))
    return out


class KvSplit:
    """The mailboxes of one (T, Hq, D) decode shape across `nranks` ranks.

    `exchange(handle_bytes) -> [handle_bytes per rank]` is how handles travel: torch.distributed.all_gather_object in a
    real run, a plain list in a single-process test where all "ranks" share one GPU (then pass `local_mailboxes`).
    """

    def __init__(self, gpu, rank, nranks, T, Hq, D, exchange=None, local_mailboxes=None):
        self.gpu, self.rank, self.nranks, self.T, self.Hq, self.D = gpu, rank, nranks, T, Hq, D
        api = gpu.api
        nbytes = int(api.need("ns_b200_kvsplit_mailbox_bytes")(nranks, T, Hq, D))
        self.opened = []
        if local_mailboxes is not None:
            self.mailbox = local_mailboxes[rank]
            ptrs = [m.ptr for m in local_mailboxes]
        else:
            self.mailbox = DevBuf(gpu, nbytes)
            self.mailbox.fill(0)
            gpu.sync()
            h = C.create_string_buffer(64)
            check(api, api.need("ns_b200_ipc_export")(gpu.raw, self.mailbox.ptr, h), "exporting the mailbox")
            handles = exchange(bytes(h.raw))
            ptrs = []
            for r, hb in enumerate(handles):
                if r == rank:
                    ptrs.append(self.mailbox.ptr)
                else:
                    p = C.c_void_p()
                    check(api, api.need("ns_b200_ipc_open")(gpu.raw, C.create_string_buffer(hb, 64), C.byref(p)), f"opening rank {r}'s mailbox")
                    self.opened.append(p.value)
                    ptrs.append(p.value)
        self.table = DevBuf.of(gpu, np.array(ptrs, dtype=np.uint64))
        self.epoch = 0

    @staticmethod
    def mailbox_bytes(api, nranks, T, Hq, D):
        return int(api.need("ns_b200_kvsplit_mailbox_bytes")(nranks, T, Hq, D))

    def scratch_floats(self, Hkv, kv_local):
        return int(self.gpu.api.need("ns_b200_kvsplit_scratch")(self.T, self.Hq, Hkv, self.D, max(1, kv_local)))

    def decode(self, q, qs, kc, vc, Hkv, kv_local, key_base, p0, scratch, epoch=None):
        """This rank's keys; pushes its partial to every mailbox under `epoch` (default: the next one)."""
        if epoch is None:
            self.epoch += 1
            epoch = self.epoch
        elif epoch == 0:
            self.device_epochs = True   # the mailbox counts the steps itself (a recorded step can be replayed)
        api = self.gpu.api

        def ptr(b):   # a rank without keys (kv_local 0) passes no caches and no scratch
            return b.ptr if b is not None else None
        check(api, api.need("ns_b200_kvsplit_decode")(self.gpu.raw, q.ptr, qs, ptr(kc), ptr(vc), self.T, self.Hq, Hkv, self.D, kv_local, key_base, p0,
                                                      ptr(scratch), self.rank, self.nranks, self.table.ptr, epoch), "ns_b200_kvsplit_decode")
        return epoch

    def step(self, q, qs, kc, vc, Hkv, kv_local, key_base, p0, scratch, out, epoch=None, wait_us=200000):
        """decode + push + combine as one kernel launch (ns_b200_kvsplit_step); epochs as `decode`."""
        if epoch is None:
            self.epoch += 1
            epoch = self.epoch
        elif epoch == 0:
            self.device_epochs = True
        api = self.gpu.api

        def ptr(b):
            return b.ptr if b is not None else None
        check(api, api.need("ns_b200_kvsplit_step")(self.gpu.raw, q.ptr, qs, ptr(kc), ptr(vc), self.T, self.Hq, Hkv, self.D, kv_local, key_base, p0,
                                                    ptr(scratch), self.rank, self.nranks, self.table.ptr, self.mailbox.ptr, epoch, wait_us, out.ptr),
              "ns_b200_kvsplit_step")
        return epoch

    def combine(self, out, epoch=None, wait_us=200000):
        api = self.gpu.api
        if epoch is None:
            epoch = 0 if getattr(self, "device_epochs", False) else self.epoch
        check(api, api.need("ns_b200_kvsplit_combine")(self.gpu.raw, self.mailbox.ptr, self.nranks, self.T, self.Hq, self.D, epoch, wait_us, out.ptr),
              "ns_b200_kvsplit_combine")

    # ---- the absorbed-MLA latent cache split the same way (a group made with D = 512 and Hq = the number of heads) -------
    def mla_scratch_floats(self, cells_local):
        return int(self.gpu.api.need("ns_b200_mla_kvsplit_scratch")(self.gpu.raw, self.T, self.Hq, max(0, cells_local)))

    def mla_decode(self, q, cache, cells_local, cell_base, pos0, scale, scratch, epoch=None):
        """This rank's cells (cache fp16 [cells_local][576]); pushes its partial to every mailbox under `epoch`."""
        if epoch is None:
            self.epoch += 1
            epoch = self.epoch
        elif epoch == 0:
            self.device_epochs = True
        api = self.gpu.api
        check(api, api.need("ns_b200_mla_kvsplit_decode")(self.gpu.raw, q.ptr, cache.ptr if cache is not None else None, self.T, self.Hq, cells_local,
                                                          cell_base, pos0, scale, scratch.ptr if scratch is not None else None, self.rank, self.nranks,
                                                          self.table.ptr, epoch), "ns_b200_mla_kvsplit_decode")
        return epoch

    def mla_combine(self, out, epoch=None, wait_us=200000):
        api = self.gpu.api
        if epoch is None:
            epoch = 0 if getattr(self, "device_epochs", False) else self.epoch
        check(api, api.need("ns_b200_mla_kvsplit_combine")(self.gpu.raw, self.mailbox.ptr, self.nranks, self.T, self.Hq, epoch, wait_us, out.ptr),
              "ns_b200_mla_kvsplit_combine")

    def close(self):
        api = self.gpu.api
        for p in self.opened:
            api.need("ns_b200_ipc_close")(self.gpu.raw, p)
        self.opened = []
