"""Datasets in the reference's preprocessed on-disk format (cafe_b200.data): the file layout and the host collate on
CPU; on the GPU the device-side collate (cafe_records_to_batch behind DeviceBatchLoader) against the host one."""
import numpy as np
import pytest


def _make_files(tmp_path, n=1000, shape="kaggle", seed=3):
    from cafe_b200 import data, dlrm_harness as H, synthetic as S
    cards, nd, s, p, *_ = H.SHAPES[shape]
    ids = S.batch_ids(cards, n, s, seed, 0).T.astype(np.int32)          # [N, F] sample-major, as on disk
    dense = S.dense_features(n, seed, 0, nd) if nd else None
    label = S.labels(n, p, seed, 0).astype(np.int32)
    data.write_record_files(tmp_path, ids, dense, label, cards)
    return data.RecordFiles(tmp_path, len(cards), nd), ids, dense, label


def test_files_round_trip_and_host_collate(tmp_path):
    from cafe_b200 import data
    files, ids, dense, label = _make_files(tmp_path, 300)
    assert len(files) == 300 and files.sparse.shape == (300, 26) and files.dense.shape == (300, 13)
    assert np.array_equal(files.counts, np.array(files.counts))
    x_int, ls_o, ls_i, t = data.host_collate(files, 10, 74)
    assert ls_i.shape == (26, 64) and ls_i.dtype.is_floating_point is False
    assert np.array_equal(ls_i.numpy(), ids[10:74].T.astype(np.int64))
    assert np.array_equal(ls_o[0].numpy(), np.arange(64))
    assert np.array_equal(x_int.numpy(), dense[10:74]) and np.array_equal(t.numpy()[:, 0], label[10:74].astype(np.float32))


def test_files_without_dense_features(tmp_path):
    from cafe_b200 import data
    files, ids, dense, label = _make_files(tmp_path, 100, "avazu")
    assert files.dense is None and files.sparse.shape == (100, 22)
    x_int, _, ls_i, _ = data.host_collate(files, 0, 100)
    assert x_int is None and np.array_equal(ls_i.numpy(), ids.T.astype(np.int64))


@pytest.mark.gpu
@pytest.mark.parametrize("shape,batch,int64", [("kaggle", 128, True), ("avazu", 96, True), ("terabyte", 257, False)])
def test_device_loader_equals_host_collate(tmp_path, shape, batch, int64):
    """Every batch, the ragged last one included, bit for bit; ids as int64 or int32."""
    import torch
    from cafe_b200 import data
    files, *_ = _make_files(tmp_path, 1000, shape)
    loader = data.DeviceBatchLoader(files, batch, "cuda", ids_int64=int64)
    assert len(loader) == (1000 + batch - 1) // batch
    lo, seen = 0, 0
    for dense, ls_o, ids, t in loader:
        hi = min(lo + batch, 1000)
        x_int, _, ls_i, t_ref = data.host_collate(files, lo, hi)
        assert ls_o is None and ids.dtype == (torch.int64 if int64 else torch.int32)
        assert torch.equal(ids.cpu().long(), ls_i) and torch.equal(t.cpu(), t_ref)
        assert (dense is None and x_int is None) or torch.equal(dense.cpu(), x_int)
        lo, seen = hi, seen + 1
    assert seen == len(loader) and lo == 1000


@pytest.mark.gpu
def test_training_from_files_equals_training_from_arrays(tmp_path):
    """The DLRM harness fed by the device loader takes the same steps as when it is fed the collated arrays."""
    import torch
    from cafe_b200 import data, dlrm_harness as H
    files, *_ = _make_files(tmp_path, 128 * 6)
    losses = []
    for source in ("files", "arrays"):
        args = H.make_parser().parse_args(["--sketch-flag", "--data-set", "kaggle", "--hash-rate", "0.3", "--sketch-alpha",
                                           "1.0000005", "--mini-batch-size", "128"])
        net = H.build_model(args, torch.device("cuda", 0))
        opt = torch.optim.SGD(H.dense_and_plain_parameters(net), lr=0.1)
        out = []
        if source == "files":
            for dense, ls_o, ids, t in data.DeviceBatchLoader(files, 128, "cuda"):
                loss, _ = H.train_step(net, opt, dense, ls_o, ids, t[:, 0])
                out.append(float(loss.detach()))
        else:
            for b in range(6):
                x_int, ls_o, ls_i, t = data.host_collate(files, b * 128, (b + 1) * 128)
                loss, _ = H.train_step(net, opt, x_int.cuda(), None, ls_i, t[:, 0].cuda())
                out.append(float(loss.detach()))
        losses.append(out)
    assert losses[0] == losses[1]
