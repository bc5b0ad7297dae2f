"""Generates module_step.npz by running the REFERENCE's own SKEmbeddingBag (tricks/sk_embedding_bag.py,
imported from the reference checkout) on CPU against the compiled reference sketch.

    python tests/golden/make_module_golden.py

One sketch field (the only case in which the reference's gradient slicing is right), threshold 3 and
no threshold re-fit, so that every lookup the sketch reports as newly hot is in the main table and the
reference's unguarded migration indexes a valid hot row.  Recorded per step: ids, the upstream
gradient, the pooled output, the importance array the reference passed to batch_insert_val, its
result, and after the last step both tables and the sketch state.
"""
import ctypes
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
from oracle.hotsketch import ReferenceSketch, reference_root  # noqa: E402

sys.path.insert(0, str(reference_root()))   # $CAFE_REFERENCE_ROOT, else `reference` beside the repository
from tricks.sk_embedding_bag import SKEmbeddingBag as RefBag  # noqa: E402

STATE_KEYS = ["main_val", "main_cnt", "main_dic", "main_flip", "lru_val", "lru_cnt", "lru_dic", "lru_t", "lru_flip",
              "queue"]


def main():
    torch.manual_seed(0)
    rng = np.random.default_rng(0)
    hotn, D, ncat, hash_size, B, steps, lr, thr = 300, 16, 5000, 40, 64, 12, 0.1, 3
    sk = ReferenceSketch(hotn, thr, 0, 1.0000005)
    wh = torch.nn.Parameter((torch.rand(hotn, D) * 2 - 1) * 0.05)
    m = RefBag(0, hotn, sk._lib, wh, "cpu", ncat, D, 0, hash_size)
    wh0, wc0 = wh.detach().clone().numpy(), m.weight_hash.detach().clone().numpy()
    opt = torch.optim.SGD([wh, m.weight_hash], lr=lr)
    real_inv = m.inv
    seen = []

    def spy(ids_p, imp_p, n):
        seen.append(np.ctypeslib.as_array(imp_p, shape=(n,)).copy())
        return real_inv(ids_p, imp_p, n)

    m.inv = spy
    offsets = torch.arange(B)
    rec = dict(ids=[], grad=[], out=[], imp=[], mask=[])
    for s in range(steps):
        ids = torch.from_numpy(np.minimum(rng.zipf(1.2, B) - 1, ncat - 1).astype(np.int64))
        g = torch.from_numpy((rng.standard_normal((B, D)) * 0.05).astype(np.float32))
        out = m(ids, offsets)
        opt.zero_grad()
        out.backward(g)
        before = sk.state()["num"]
        m.insert_grad(ids)
        opt.step()
        rec["ids"].append(ids.numpy())
        rec["grad"].append(g.numpy())
        rec["out"].append(out.detach().numpy())
        rec["imp"].append(seen[-1])
        rec["mask"].append(np.int32(sk.state()["num"] - before))
    st = sk.state()
    np.savez_compressed(HERE / "module_step.npz", hotn=hotn, D=D, ncat=ncat, hash_size=hash_size, lr=lr, thr=thr,
                        wh0=wh0, wc0=wc0, wh=wh.detach().numpy(), wc=m.weight_hash.detach().numpy(),
                        ids=np.stack(rec["ids"]), grad=np.stack(rec["grad"]), out=np.stack(rec["out"]),
                        imp=np.stack(rec["imp"]), newhot=np.array(rec["mask"]),
                        scalars=np.array([st["thr_bits"], st["real_n"], st["num"], st["t"], st["gflip"]], np.int64),
                        **{k: st[k] for k in STATE_KEYS})
    print("steps", steps, "newly hot per step", rec["mask"], "hot rows in use", st["num"])


if __name__ == "__main__":
    main()
