"""Embedding objectives: InfoNCE, its chunked form, Matryoshka prefixes, cross-rank negatives, pooling."""
import torch

from paddleformers_b200.nn.contrastive import (InfClLoss, MatryoshkaContrastiveLoss, MatryoshkaInfClLoss, SimpleContrastiveLoss,
                                               gather_with_gradient, pool_embeddings)


def test_chunked_loss_equals_the_dense_one_in_value_and_gradient():
    torch.manual_seed(0)
    q = torch.nn.functional.normalize(torch.randn(6, 16), dim=-1).requires_grad_(True)
    p = torch.nn.functional.normalize(torch.randn(18, 16), dim=-1).requires_grad_(True)      # 3 passages per query
    dense = SimpleContrastiveLoss(0.05)(q, p)
    gq, gp = torch.autograd.grad(dense, (q, p))
    # hand-written reference: -log softmax at the positive column i * 3
    sc = (q @ p.t()) / 0.05
    want = -(sc.log_softmax(-1)[torch.arange(6), torch.arange(6) * 3]).mean()
    torch.testing.assert_close(dense, want)
    for chunk in (4, 5, 18, 64):
        loss = InfClLoss(0.05, chunk=chunk)(q, p)
        cq, cp = torch.autograd.grad(loss, (q, p))
        torch.testing.assert_close(loss, dense, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(cq, gq, rtol=1e-4, atol=1e-6)
        torch.testing.assert_close(cp, gp, rtol=1e-4, atol=1e-6)
    # Matryoshka: sum over re-normalised prefixes; no dims = the plain loss
    m = MatryoshkaContrastiveLoss(0.05, [4, 8, 16])(q, p)
    parts = sum(SimpleContrastiveLoss(0.05)(torch.nn.functional.normalize(q[:, :d], dim=-1), torch.nn.functional.normalize(p[:, :d], dim=-1))
                for d in (4, 8, 16))
    torch.testing.assert_close(m, parts)
    torch.testing.assert_close(MatryoshkaInfClLoss(0.05, [4, 8, 16], chunk=7)(q, p), m, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(MatryoshkaContrastiveLoss(0.05)(q, p), dense)


def test_pooling_handles_left_and_right_padding():
    h = torch.arange(2 * 4 * 3, dtype=torch.float32).view(2, 4, 3)
    right = torch.tensor([[1, 1, 1, 0], [1, 1, 0, 0]])
    out = pool_embeddings(h, right, "last", normalize=False)
    assert torch.equal(out, torch.stack([h[0, 2], h[1, 1]]))
    left = torch.tensor([[0, 1, 1, 1], [0, 0, 1, 1]])
    assert torch.equal(pool_embeddings(h, left, "last", normalize=False), torch.stack([h[0, 3], h[1, 3]]))
    mean = pool_embeddings(h, right, "mean", normalize=False)
    torch.testing.assert_close(mean[1], h[1, :2].mean(0))
    assert torch.allclose(pool_embeddings(h, right).norm(dim=-1), torch.ones(2))


def _gather_worker(rank, world):
    import torch.distributed as dist

    torch.manual_seed(0)
    q_all = torch.nn.functional.normalize(torch.randn(4, 8), dim=-1)
    p_all = torch.nn.functional.normalize(torch.randn(4, 8), dim=-1)
    q = q_all[rank * 2:(rank + 1) * 2].clone().requires_grad_(True)
    p = p_all[rank * 2:(rank + 1) * 2].clone().requires_grad_(True)
    # each rank: its own queries against the passages of all ranks; positives sit at the global row of the local passage
    allp = gather_with_gradient(p)
    scores = (q @ allp.t()) / 0.1
    target = torch.arange(2) + rank * 2
    loss = torch.nn.functional.cross_entropy(scores, target, reduction="sum") / 4       # global mean, this rank's share
    loss.backward()
    total = loss.detach().clone()
    dist.all_reduce(total)
    return total.item(), q.grad, p.grad


def test_cross_rank_negatives_give_the_single_process_gradients():
    from dist_utils import run_distributed

    res = run_distributed(_gather_worker, 2)
    torch.manual_seed(0)
    q = torch.nn.functional.normalize(torch.randn(4, 8), dim=-1).requires_grad_(True)
    p = torch.nn.functional.normalize(torch.randn(4, 8), dim=-1).requires_grad_(True)
    loss = SimpleContrastiveLoss(0.1)(q, p)
    loss.backward()
    assert abs(res[0][0] - loss.item()) < 1e-5
    torch.testing.assert_close(torch.cat([res[0][1], res[1][1]]), q.grad, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(torch.cat([res[0][2], res[1][2]]), p.grad, rtol=1e-5, atol=1e-6)
