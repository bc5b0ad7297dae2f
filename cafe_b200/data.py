"""Datasets in the reference's preprocessed on-disk format, batched on the device.

The reference's loaders memory-map four files per dataset (ArtifactEvaluation/load_data.py:44-66; the same arrays
behind dlrm_data_pytorch.py:643-649):

    processed_sparse_sep.bin   int32   [N, F]   categorical ids, sample-major
    processed_dense.bin        float32 [N, Dn]  dense features (absent for Avazu-like data, Dn = 0)
    processed_label.bin        int32   [N]
    processed_count.bin        int32   [F]      cardinality of every field

and collate every batch on the host into one int64 index tensor per field (dlrm_data_pytorch.py:395-437), which the
training loop then moves to the device field by field.  `DeviceBatchLoader` copies a block of rows as it lies on
disk (pinned staging buffers, a copy stream, two batches in flight) and transposes it on the device with
cafe_records_to_batch; it yields (dense [B, Dn] or None, offsets None, ids [F, B] int64, labels [B, 1] float32) on
the device, the tuple the reference's collate functions return, with arange(B) offsets implied (one id per bag).
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from . import _lib

FILES = ("processed_sparse_sep.bin", "processed_dense.bin", "processed_label.bin", "processed_count.bin")


class RecordFiles:
    """The four memory-mapped arrays of one dataset directory."""

    def __init__(self, path, num_sparse: int, num_dense: int):
        p = Path(path)
        self.num_sparse, self.num_dense = int(num_sparse), int(num_dense)
        self.label = np.memmap(p / FILES[2], dtype=np.int32, mode="r")
        self.num_sample = int(self.label.shape[0])
        self.sparse = np.memmap(p / FILES[0], dtype=np.int32, mode="r").reshape(self.num_sample, self.num_sparse)
        self.dense = (np.memmap(p / FILES[1], dtype=np.float32, mode="r").reshape(self.num_sample, self.num_dense)
                      if self.num_dense else None)
        self.counts = np.fromfile(p / FILES[3], dtype=np.int32).reshape(self.num_sparse)

    def __len__(self):
        return self.num_sample


def write_record_files(path, sparse: np.ndarray, dense, label: np.ndarray, counts) -> None:
    """Writes arrays in the reference's format (used to build datasets from synthetic data and by the tests)."""
    p = Path(path)
    p.mkdir(parents=True, exist_ok=True)
    np.ascontiguousarray(sparse, np.int32).tofile(p / FILES[0])
    if dense is not None:
        np.ascontiguousarray(dense, np.float32).tofile(p / FILES[1])
    np.ascontiguousarray(label, np.int32).tofile(p / FILES[2])
    np.ascontiguousarray(counts, np.int32).tofile(p / FILES[3])


def host_collate(files: RecordFiles, lo: int, hi: int):
    """The reference's collate on the host (dlrm_data_pytorch.py:411-424), for comparison."""
    x_cat = torch.tensor(np.array(files.sparse[lo:hi]), dtype=torch.long)
    x_int = torch.tensor(np.array(files.dense[lo:hi]), dtype=torch.float) if files.dense is not None else None
    t = torch.tensor(np.array(files.label[lo:hi]), dtype=torch.float32).view(-1, 1)
    ls_i = torch.stack([x_cat[:, i] for i in range(x_cat.shape[1])])
    ls_o = torch.stack([torch.arange(x_cat.shape[0]) for _ in range(x_cat.shape[1])])
    return x_int, ls_o, ls_i, t


class DeviceBatchLoader:
    """Iterates over consecutive batches of `files` (rows [start, stop)), collated on the device."""

    def __init__(self, files: RecordFiles, batch: int, device="cuda", start: int = 0, stop: int | None = None,
                 drop_last: bool = False, ids_int64: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("DeviceBatchLoader needs a CUDA device")
        self.files, self.B = files, int(batch)
        self.device = torch.device(device)
        self.start, self.stop = int(start), int(len(files) if stop is None else stop)
        self.drop_last, self.ids_int64 = drop_last, ids_int64
        self.lib = _lib.load()
        F, Dn = files.num_sparse, files.num_dense
        with torch.cuda.device(self.device):
            self.copy_stream = torch.cuda.Stream()
            self.slots = []
            for _ in range(2):
                self.slots.append(dict(
                    h_sparse=torch.empty(self.B, F, dtype=torch.int32).pin_memory(),
                    h_dense=torch.empty(self.B, max(Dn, 1), dtype=torch.float32).pin_memory(),
                    h_label=torch.empty(self.B, dtype=torch.int32).pin_memory(),
                    d_sparse=torch.empty(self.B, F, dtype=torch.int32, device=self.device),
                    d_label=torch.empty(self.B, dtype=torch.int32, device=self.device),
                    ready=torch.cuda.Event(), free=torch.cuda.Event()))

    def __len__(self):
        n = self.stop - self.start
        return n // self.B if self.drop_last else (n + self.B - 1) // self.B

    def _stage(self, slot, lo, hi):
        """Host copy into the pinned buffers, then the H2D copies on the copy stream."""
        n = hi - lo
        f = self.files
        slot["free"].synchronize()          # the kernels that read this slot's device buffers have run
        slot["h_sparse"][:n].numpy()[...] = f.sparse[lo:hi]
        slot["h_label"][:n].numpy()[...] = f.label[lo:hi]
        dense = None
        with torch.cuda.stream(self.copy_stream):
            slot["d_sparse"][:n].copy_(slot["h_sparse"][:n], non_blocking=True)
            slot["d_label"][:n].copy_(slot["h_label"][:n], non_blocking=True)
            if f.dense is not None:
                slot["h_dense"][:n].numpy()[...] = f.dense[lo:hi]
                dense = slot["h_dense"][:n].to(self.device, non_blocking=True)
            slot["ready"].record(self.copy_stream)
        slot["n"], slot["dense"] = n, dense

    def _finish(self, slot):
        """On the caller's stream: wait for the copies, transpose on the device."""
        n, F = slot["n"], self.files.num_sparse
        main = torch.cuda.current_stream(self.device)
        main.wait_event(slot["ready"])
        ids = torch.empty(F, n, dtype=torch.int64 if self.ids_int64 else torch.int32, device=self.device)
        labels = torch.empty(n, 1, dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cafe_records_to_batch(slot["d_sparse"].data_ptr(), n, F, ids.data_ptr(), int(self.ids_int64),
                                                      slot["d_label"].data_ptr(), labels.data_ptr(), main.cuda_stream),
                       "cafe_records_to_batch")
        slot["free"].record(main)
        dense = slot["dense"]
        if dense is not None:
            dense.record_stream(main)
        return dense, None, ids, labels

    def __iter__(self):
        bounds = []
        lo = self.start
        while lo < self.stop:
            hi = min(lo + self.B, self.stop)
            if hi - lo < self.B and self.drop_last:
                break
            bounds.append((lo, hi))
            lo = hi
        with torch.cuda.device(self.device):
            if bounds:
                self._stage(self.slots[0], *bounds[0])
            for i in range(len(bounds)):
                if i + 1 < len(bounds):
                    self._stage(self.slots[(i + 1) % 2], *bounds[i + 1])   # the next batch travels while this one is used
                yield self._finish(self.slots[i % 2])
