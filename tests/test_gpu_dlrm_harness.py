"""The DLRM / DCN harness (cafe_b200.dlrm_harness) against the same model on the CPU reference path.

Both sides build the dense part from the same seed (bottom / top MLP, dot interaction or cross + deep head, BCE
loss, SGD, all stock PyTorch); the embedding side is the product (SKEmbeddingGroup for the sketch fields, plain
EmbeddingBags for the small fields) on the GPU and, on the CPU, the restatement of the reference's module step
(oracle.ModuleOracle over the C sketch oracle) plus torch CPU EmbeddingBags with identical initial tables.
Importances are computed independently on each side (fp32 sums in a different order), so a threshold decision may
differ by an ulp here and there; the curves must agree within the tolerances stated at each test."""
import copy

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


class OracleEmbeddingLayer:
    """CPU mirror of dlrm_harness.CafeEmbeddingLayer: same forward signature, ModuleOracle for the sketch fields."""

    def __init__(self, gpu_layer, thr=1, adjust=1, alpha=1.0000005):
        import torch
        from oracle.hotsketch import OracleSketch
        from oracle.module_oracle import ModuleOracle
        self.device = torch.device("cpu")
        self.sketch_fields, self.plain_fields = gpu_layer.sketch_fields, gpu_layer.plain_fields
        self.group, self.orc = None, None
        if gpu_layer.group is not None:
            g = gpu_layer.group
            self.sk = OracleSketch(g.hotn, thr, adjust, alpha)
            self.orc = ModuleOracle(self.sk, g.weight_high.detach().cpu().numpy(), [w.detach().cpu().numpy() for w in g.weight_hash],
                                    g.f_offsets, g.hash_sizes)
        self.plain = copy.deepcopy(gpu_layer.plain).to("cpu")
        self.lr = 0.1
        self._e = None

    def set_lr(self, lr):
        self.lr = float(lr)

    def parameters(self):
        return self.plain.parameters()

    def __call__(self, lS_o, lS_i, test=False):
        import torch
        ids = lS_i.numpy()
        F, B = ids.shape
        cols = [None] * F
        self._ids = ids
        if self.orc is not None:
            self._e = torch.from_numpy(self.orc.forward(ids[self.sketch_fields])).requires_grad_(True)
            for j, i in enumerate(self.sketch_fields):
                cols[i] = self._e[:, j, :]
        ar = torch.arange(B)
        for j, i in enumerate(self.plain_fields):
            cols[i] = self.plain[j](lS_i[i], ar)
        return torch.stack(cols, dim=1)

    def after_backward(self):
        if self.orc is not None:
            self.orc.backward(self._ids[self.sketch_fields], self._e.grad.numpy(), self.lr)


def _mirror(net):
    """The GPU net's dense modules copied to the CPU around an OracleEmbeddingLayer."""
    emb = net.emb
    net.emb = None
    cpu = copy.deepcopy(net).to("cpu")
    net.emb = emb
    del cpu._modules["emb"]
    cpu.__dict__["emb"] = OracleEmbeddingLayer(emb)   # not a Module: its tables are numpy arrays
    return cpu


def _run_pair(shape, model, cr, hr, B, steps, lr, dim=None, bot=None, top=None):
    import torch
    from cafe_b200 import dlrm_harness as H
    args = H.make_parser().parse_args(["--sketch-flag", "--data-set", shape, "--model", model, "--compress-rate", str(cr),
                                       "--hash-rate", str(hr), "--sketch-alpha", "1.0000005", "--mini-batch-size", str(B),
                                       "--learning-rate", str(lr)] + (["--arch-sparse-feature-size", str(dim)] if dim else []) +
                                      (["--arch-mlp-bot", bot] if bot else []) + (["--arch-mlp-top", top] if top else []))
    net = H.build_model(args, torch.device("cuda", 0))
    cpu = _mirror(net)
    gopt = torch.optim.SGD(H.dense_and_plain_parameters(net), lr=lr)
    copt = torch.optim.SGD([p for n, p in cpu.named_parameters()] + list(cpu.emb.parameters()), lr=lr)
    gl, cl, gp, cp, ys = [], [], [], [], []
    for s in range(steps):
        dense, lS_o, ids, y = H.synthetic_batch(shape, B, 2024, s, "cuda")
        loss, z = H.train_step(net, gopt, dense, lS_o, ids, y)
        gl.append(float(loss.detach()))
        gp.append(z.detach().squeeze(1).cpu().numpy())
        # CPU reference path, the reference's step order: forward, loss, zero_grad, backward, insert_grad (importance ->
        # insert -> migration) and SGD
        cpu.emb.set_lr(lr)
        zc = cpu(dense.cpu() if dense is not None else None, lS_o, ids, False)
        lc = torch.nn.functional.binary_cross_entropy(zc.squeeze(1), y.cpu())
        copt.zero_grad()
        lc.backward()
        cpu.emb.after_backward()
        copt.step()
        cl.append(float(lc.detach()))
        cp.append(zc.detach().squeeze(1).numpy())
        ys.append(y.cpu().numpy())
    return net, cpu, np.array(gl), np.array(cl), gp, cp, ys


def _hot_ids(state):
    return set(state["main_val"][state["main_dic"] != 0].tolist())


def test_kaggle_configuration_loss_and_auc_curves():
    """configs[0]: 26 Kaggle-shaped fields, dim 16, bottom 13-512-256-64-16, top 512-256-1, batch 128, SGD 0.1,
    compress 0.001 / hash-rate 0.3, 600 steps.  Tolerances: |loss difference| per step < 5e-3 (BCE mean over 128
    samples), AUC over the last 150 steps within 0.01, hot sets within 5 % (every threshold decision that falls the
    other way on one side moves an id in or out of the hot set for good, and 600 steps x 26 calls accumulate them)."""
    from cafe_b200 import dlrm_harness as H
    net, cpu, gl, cl, gp, cp, ys = _run_pair("kaggle", "dlrm", 0.001, 0.3, 128, 600, 0.1)
    assert len(net.emb.sketch_fields) == 26 and net.emb.hotn == 13505
    assert np.max(np.abs(gl - cl)) < 5e-3, (float(np.max(np.abs(gl - cl))), gl[-3:], cl[-3:])
    yy = np.concatenate(ys[-150:])
    a_g, a_c = H.auc(yy, np.concatenate(gp[-150:])), H.auc(yy, np.concatenate(cp[-150:]))
    assert abs(a_g - a_c) < 0.01, (a_g, a_c)
    hg, hc = _hot_ids(net.emb.group.sketch.state()), _hot_ids(cpu.emb.sk.state())
    assert len(hg ^ hc) <= 0.05 * max(1, len(hc)), (len(hg), len(hc), len(hg ^ hc))


def test_avazu_dcn_configuration_sketch_and_plain_fields():
    """configs[4]: DCN head (3 cross layers, deep 1024-1024) over 22 Avazu-shaped fields, dim 16, batch 4096,
    compress 0.1 / hash-rate 0.7: 9 fields go through the sketch, 13 keep plain tables.  30 steps; per-step loss
    within 5e-3."""
    net, cpu, gl, cl, gp, cp, ys = _run_pair("avazu", "dcn", 0.1, 0.7, 4096, 30, 0.1)
    assert len(net.emb.sketch_fields) == 9 and len(net.emb.plain_fields) == 13 and net.emb.hotn == 161986
    assert np.max(np.abs(gl - cl)) < 5e-3, (float(np.max(np.abs(gl - cl))), gl[-3:], cl[-3:])
    for a, b in zip(net.emb.plain, cpu.emb.plain):
        np.testing.assert_allclose(a.weight.detach().cpu().numpy(), b.weight.detach().numpy(), rtol=1e-4, atol=1e-6)


def test_terabyte_configuration_few_steps():
    """configs[2]: Terabyte-shaped fields, dim 128, bottom 13-512-256-128, top 1024-1024-512-256-1, batch 2048,
    compress 0.001 / hash-rate 0.3.  12 steps; per-step loss within 5e-3."""
    net, cpu, gl, cl, gp, cp, ys = _run_pair("terabyte", "dlrm", 0.001, 0.3, 2048, 12, 0.1)
    assert net.emb.hotn == 120171
    assert np.max(np.abs(gl - cl)) < 5e-3, (float(np.max(np.abs(gl - cl))), gl, cl)
