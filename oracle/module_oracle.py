"""numpy restatement of the SKEmbeddingBag step.  TEST INFRASTRUCTURE ONLY.

Follows the reference's pieces in the order its training loop runs them:
  forward      tricks/sk_embedding_bag.py:101-152  (query -> two gathers -> where)
  importance   tricks/sk_embedding_bag.py:178-189  (norm of each lookup's gradient row * N / sum)
  insert       tricks/sketch.cpp:281-296           (through a sketch oracle object)
  migration    tricks/sk_embedding_bag.py:199-208  (guarded: only when the post-insert query is hot)
  SGD          dlrm_s_pytorch.py:1658              (rows chosen at forward time, lr * summed gradient)
The sketch is any object with batch_query / batch_insert_val (OracleSketch or ReferenceSketch).

Parity status: the arithmetic above is restated from the reference's Python; it is pinned by
tests/golden/module_step.npz, produced by running the reference's own SKEmbeddingBag class on CPU
(tests/golden/make_module_golden.py).
"""
from __future__ import annotations

import numpy as np


class ModuleOracle:
    def __init__(self, sketch, weight_high, weight_hash, f_offsets, hash_sizes):
        self.sk = sketch
        self.wh = np.array(weight_high, np.float32, copy=True)
        self.wc = [np.array(w, np.float32, copy=True) for w in weight_hash]
        self.off = [int(o) for o in f_offsets]
        self.hs = [int(h) for h in hash_sizes]
        self.hotn = self.wh.shape[0]
        self.F = len(self.wc)

    def gids(self, ids):
        return [((ids[f].astype(np.int64) + self.off[f]) & 0xFFFFFFFF).astype(np.uint32) for f in range(self.F)]

    def forward(self, ids):
        """ids [F,B] local ids -> out [B,F,D]; remembers the row choice for the update."""
        g = self.gids(ids)
        B = ids.shape[1]
        out = np.empty((B, self.F, self.wh.shape[1]), np.float32)
        self.rows = []
        for f in range(self.F):
            q = self.sk.batch_query(g[f])
            hot = q < 0
            dic = np.abs(q.astype(np.int64))
            hi = self.wh[dic % self.hotn]
            lo = self.wc[f][dic % self.hs[f]]
            out[:, f] = np.where(hot[:, None], hi, lo)
            self.rows.append((hot, dic % self.hotn, dic % self.hs[f]))
        self.last_gids = g
        return out

    @staticmethod
    def importance(grad_f):
        """grad_f [B,D] -> float32 [B] (tricks/sk_embedding_bag.py:178-189)."""
        n = np.sqrt((grad_f.astype(np.float32) ** 2).sum(axis=1, dtype=np.float32)).astype(np.float32)
        return (n * np.float32(len(n)) / n.sum(dtype=np.float32)).astype(np.float32)

    def backward(self, ids, grad, lr, importance=None):
        """grad [B,F,D].  `importance` [F,B] overrides the computed one (bit-exact sketch comparisons
        feed both sides the same floats).  Returns (masks [F,B], migrated count)."""
        masks, migrated = [], 0
        for f in range(self.F):
            imp = self.importance(grad[:, f]) if importance is None else np.asarray(importance[f], np.float32)
            m = self.sk.batch_insert_val(self.last_gids[f], imp)
            q = self.sk.batch_query(self.last_gids[f])
            for x in np.nonzero(m)[0]:
                if q[x] < 0:   # guard: the reference indexes weight_h[global id] otherwise
                    self.wh[-q[x]] = self.wc[f][int(ids[f][x]) % self.hs[f]]
                    migrated += 1
            masks.append(m)
        lr = np.float32(lr)
        gh = np.zeros_like(self.wh)
        for f in range(self.F):
            hot, rh, rc = self.rows[f]
            gf = grad[:, f].astype(np.float32)
            np.add.at(gh, rh[hot], gf[hot])
            gc = np.zeros_like(self.wc[f])
            np.add.at(gc, rc[~hot], gf[~hot])
            self.wc[f] -= lr * gc
        self.wh -= lr * gh
        return np.stack(masks), migrated
