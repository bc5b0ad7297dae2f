"""Loss / AUC curve parity of a small DLRM-shaped model trained with the CUDA CAFE embeddings against the
same model trained with the CPU restatement of the reference's module step.

Dense part (bottom MLP, dot interaction, top MLP, BCE loss, SGD) is stock PyTorch on both sides with identical
initial weights; the embedding side is cafe_b200.SKEmbeddingGroup on the GPU and oracle.ModuleOracle (+ the C
sketch oracle) on the CPU.  Importances are computed independently on each side (fp32, different summation
order), so threshold decisions may differ by an ulp here and there; the curves must still agree within the
tolerances below."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LOSS_ATOL = 2e-3      # per-step training loss (BCE, mean) -- absolute
AUC_ATOL = 0.01       # ROC-AUC over the last 40 steps' predictions


def _dense(dev, D, F, seed):
    import torch
    torch.manual_seed(seed)
    bot = torch.nn.Sequential(torch.nn.Linear(13, 32), torch.nn.ReLU(), torch.nn.Linear(32, D), torch.nn.ReLU())
    n_int = (F + 1) * F // 2 + D
    top = torch.nn.Sequential(torch.nn.Linear(n_int, 32), torch.nn.ReLU(), torch.nn.Linear(32, 1))
    return bot.to(dev), top.to(dev)


def _interact(x, emb):
    import torch
    B, D = x.shape
    T = torch.cat([x.unsqueeze(1), emb], dim=1)            # [B, F+1, D]
    Z = torch.bmm(T, T.transpose(1, 2))
    li, lj = torch.tril_indices(T.shape[1], T.shape[1], offset=-1)
    return torch.cat([x, Z[:, li, lj]], dim=1)


def _auc(y, p):
    order = np.argsort(p)
    y = y[order]
    n1 = y.sum()
    n0 = len(y) - n1
    if n1 == 0 or n0 == 0:
        return 0.5
    ranks = np.arange(1, len(y) + 1)
    return float((ranks[y == 1].sum() - n1 * (n1 + 1) / 2) / (n0 * n1))


def test_loss_and_auc_curves_match_cpu_reference_path():
    import torch
    import cafe_b200
    from cafe_b200 import synthetic as S
    from oracle.hotsketch import OracleSketch
    from oracle.module_oracle import ModuleOracle
    cards = [1460, 583, 1013122, 220260, 305, 12517, 93145, 835159]
    F, D, B, steps, lr = len(cards), 16, 128, 120, 0.1
    grp = cafe_b200.SKEmbeddingGroup(cards, D, 0.01, 0.3, 1, 1, 1.0000005, device="cuda", max_batch=B, lr=lr, seed=5)
    sk = OracleSketch(grp.hotn, 1, 1, 1.0000005)
    orc = ModuleOracle(sk, grp.weight_high.detach().cpu().numpy(), [w.detach().cpu().numpy() for w in grp.weight_hash],
                       grp.f_offsets, grp.hash_sizes)
    gbot, gtop = _dense("cuda", D, F, 1)
    cbot, ctop = _dense("cpu", D, F, 1)
    gopt = torch.optim.SGD(list(gbot.parameters()) + list(gtop.parameters()), lr=lr)
    copt = torch.optim.SGD(list(cbot.parameters()) + list(ctop.parameters()), lr=lr)
    lossf = torch.nn.BCEWithLogitsLoss()
    gl, cl, gp, cp, ys = [], [], [], [], []
    # labels depend on the ids so that there is something to learn
    wtrue = np.random.default_rng(0).standard_normal(F)
    for s in range(steps):
        ids = S.batch_ids(cards, B, 1.1, 2024, s)
        dense = S.dense_features(B, 2024, s)
        signal = ((ids % 7 == 0).astype(np.float32).T @ wtrue).astype(np.float32)
        y = (signal + 0.3 * np.random.default_rng(s).standard_normal(B) > 0).astype(np.float32)
        # --- GPU: product path
        emb = grp(torch.from_numpy(ids))
        logit = gtop(_interact(gbot(torch.from_numpy(dense).cuda()), emb)).squeeze(1)
        loss = lossf(logit, torch.from_numpy(y).cuda())
        gopt.zero_grad()
        loss.backward()
        gopt.step()
        gl.append(float(loss))
        gp.append(torch.sigmoid(logit).detach().cpu().numpy())
        # --- CPU: restatement of the reference path
        e = torch.from_numpy(orc.forward(ids)).requires_grad_(True)
        logit_c = ctop(_interact(cbot(torch.from_numpy(dense)), e)).squeeze(1)
        loss_c = lossf(logit_c, torch.from_numpy(y))
        copt.zero_grad()
        loss_c.backward()
        copt.step()
        orc.backward(ids, e.grad.numpy(), lr)
        cl.append(float(loss_c))
        cp.append(torch.sigmoid(logit_c).detach().numpy())
        ys.append(y)
    gl, cl = np.array(gl), np.array(cl)
    assert np.max(np.abs(gl - cl)) < LOSS_ATOL, (np.max(np.abs(gl - cl)), gl[-5:], cl[-5:])
    assert cl[-20:].mean() < cl[:20].mean()                     # the model does learn
    yy = np.concatenate(ys[-40:])
    a_g, a_c = _auc(yy, np.concatenate(gp[-40:])), _auc(yy, np.concatenate(cp[-40:]))
    assert abs(a_g - a_c) < AUC_ATOL, (a_g, a_c)
    # the hot sets stay (nearly) identical: same hot rows handed out
    sg, sc = grp.sketch.state(), sk.state()
    hot_g = set(sg["main_val"][sg["main_dic"] != 0].tolist())
    hot_c = set(sc["main_val"][sc["main_dic"] != 0].tolist())
    assert len(hot_g ^ hot_c) <= 0.02 * max(1, len(hot_c)), (len(hot_g), len(hot_c), len(hot_g ^ hot_c))
