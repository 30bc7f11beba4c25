"""CPU-side asynchronous LoRA hand-off through POSIX shared memory.

Keeps the protocol of the reference's loader processes (load_lora_shm_multi.py:47-121) and of the readers
(sdxl_unet_server.py:159-181, pipeline_controlnet_sd_xl_katz.py:254-280,1527-1555,1772-1777):

  * one int8 flag per loader in the segment `start_loading_flag`: 0 idle, 1..9 "load adapter number <code>",
    10 loaded, 100 quit;
  * one fp16 segment per LoRA tensor, named `<tensor key>_<loader id>`, with the shapes of the adapter's info file
    (lora_info_shm/<repo>.json: {key: {"shape", "nbytes"}});
  * the reader polls the flags, and when they sum to 10 * n_loaders copies the tensors out and clears the segments.

Differences from the reference: every wait is bounded (a dead peer raises instead of hanging the job; the reference
busy-waits forever, load_lora_shm_multi.py:85-99), adapters are gathered per loader (so ranks 64 and 32 can be merged
as sum_i B_i A_i instead of the reference's element-wise sum of A's and B's, sdxl_unet_server.py:169-173), and an
optional name prefix keeps concurrent jobs apart.
"""
import time
from collections import OrderedDict
from multiprocessing import shared_memory

import numpy as np
import torch

from ._lib import KatzError

FLAG_IDLE, FLAG_DONE, FLAG_QUIT = 0, 10, 100
FLAG_SEGMENT = "start_loading_flag"


def _seg_name(prefix, key, loader_id):
    return "%s%s_%d" % (prefix, key, loader_id)


def _attach(name, create, size):
    if create:
        try:
            return shared_memory.SharedMemory(name=name, create=True, size=size)
        except FileExistsError:
            old = shared_memory.SharedMemory(name=name)      # a leaked segment of a dead job: reuse it
            if old.size < size:
                old.close()
                old.unlink()
                return shared_memory.SharedMemory(name=name, create=True, size=size)
            return old
    return shared_memory.SharedMemory(name=name)


class _Segments:
    def __init__(self, info, loader_id, prefix, create):
        self.shm, self.np = OrderedDict(), OrderedDict()
        for key, meta in info.items():
            shape = tuple(meta["shape"])
            nbytes = int(meta.get("nbytes", int(np.prod(shape)) * 2))
            s = _attach(_seg_name(prefix, key, loader_id), create, nbytes)
            self.shm[key] = s
            self.np[key] = np.ndarray(shape, dtype=np.float16, buffer=s.buf)

    def close(self, unlink):
        self.np.clear()
        for s in self.shm.values():
            s.close()
            if unlink:
                try:
                    s.unlink()
                except FileNotFoundError:
                    pass
        self.shm.clear()


class LoraShmLoader:
    """One loader process (load_lora_shm_multi.py). `source(code)` returns {key: fp16 array-like} for request `code`."""

    def __init__(self, loader_id, loader_num, info, source, prefix=""):
        self.loader_id, self.loader_num, self.source, self.prefix = loader_id, loader_num, source, prefix
        self.flag_shm = _attach(prefix + FLAG_SEGMENT, loader_id == 0, loader_num)
        self.flags = np.ndarray((loader_num,), dtype=np.int8, buffer=self.flag_shm.buf)
        self.flags[loader_id] = FLAG_IDLE
        self.seg = _Segments(info, loader_id, prefix, create=True)
        for a in self.seg.np.values():
            a[...] = 0

    def serve(self, idle_timeout_s=600.0, poll_s=0.0005):
        """Serve load requests until the quit flag; raises KatzError after `idle_timeout_s` without a request."""
        served = 0
        while True:
            t0 = time.time()
            while True:
                state = int(self.flags[self.loader_id])
                if state not in (FLAG_IDLE, FLAG_DONE):
                    break
                if time.time() - t0 > idle_timeout_s:
                    raise KatzError("LoRA loader %d: no request for %.0f s" % (self.loader_id, idle_timeout_s))
                time.sleep(poll_s)
            if state == FLAG_QUIT:
                return served
            tensors = self.source(state)
            for key, arr in tensors.items():
                dst = self.seg.np[key]
                src = arr.numpy() if torch.is_tensor(arr) else np.asarray(arr)
                if src.shape != dst.shape:
                    raise KatzError("LoRA tensor %s has shape %s, segment has %s" % (key, src.shape, dst.shape))
                dst[...] = src
            self.flags[self.loader_id] = FLAG_DONE
            served += 1

    def close(self):
        self.flags = None
        self.seg.close(unlink=True)
        self.flag_shm.close()
        if self.loader_id == 0:
            try:
                self.flag_shm.unlink()
            except FileNotFoundError:
                pass


class LoraShmClient:
    """The GPU process's side: raise the request flags, poll, gather to the device, clear."""

    def __init__(self, infos, prefix="", attach_timeout_s=60.0):
        """infos: one info dict per loader (loader i serves infos[i])."""
        self.prefix, self.n = prefix, len(infos)
        t0 = time.time()
        while True:
            try:
                self.flag_shm = shared_memory.SharedMemory(name=prefix + FLAG_SEGMENT)
                self.segs = [_Segments(info, i, prefix, create=False) for i, info in enumerate(infos)]
                break
            except FileNotFoundError:
                if time.time() - t0 > attach_timeout_s:
                    raise KatzError("LoRA loader segments did not appear within %.0f s" % attach_timeout_s)
                time.sleep(0.05)
        self.flags = np.ndarray((self.n,), dtype=np.int8, buffer=self.flag_shm.buf)
        self._pinned = {}

    def request(self, codes):
        """codes[i] in 1..9 asks loader i for its adapter number codes[i] (…katz.py:1174-1184)."""
        for i, c in enumerate(codes):
            if not 1 <= int(c) <= 9:
                raise KatzError("load request codes are 1..9")
            self.flags[i] = int(c)

    def status(self):
        """Sum of the flags: the value the reference ships to the UNet server every step (…katz.py:1527-1532)."""
        return int(self.flags.astype(np.int32).sum())

    def ready(self):
        return self.status() == FLAG_DONE * self.n

    def wait(self, timeout_s=120.0, poll_s=0.0005):
        t0 = time.time()
        while not self.ready():
            if time.time() - t0 > timeout_s:
                raise KatzError("LoRA loaders not done after %.0f s (flags %s)" % (timeout_s, self.flags.tolist()))
            time.sleep(poll_s)

    def gather(self, loader_id, device, dtype=torch.float16):
        """{key: tensor on `device`} for one loader: a pinned staging copy per tensor, then asynchronous H2D copies."""
        if int(self.flags[loader_id]) != FLAG_DONE:
            raise KatzError("loader %d has not finished (flag %d)" % (loader_id, int(self.flags[loader_id])))
        out = OrderedDict()
        for key, arr in self.segs[loader_id].np.items():
            pk = (loader_id, key)
            pin = self._pinned.get(pk)
            if pin is None:
                pin = torch.empty(arr.shape, dtype=torch.float16)
                if torch.cuda.is_available():
                    pin = pin.pin_memory()
                self._pinned[pk] = pin
            pin.numpy()[...] = arr
            out[key] = pin.to(device=device, dtype=dtype, non_blocking=True)
        return out

    def clear(self):
        """clear_shm (…katz.py:1772-1777): zero the tensors and return the loaders to idle."""
        for i, seg in enumerate(self.segs):
            for a in seg.np.values():
                a[...] = 0
            self.flags[i] = FLAG_IDLE

    def quit(self):
        for i in range(self.n):
            self.flags[i] = FLAG_QUIT

    def close(self):
        self.flags = None
        for s in self.segs:
            s.close(unlink=False)
        self.flag_shm.close()
