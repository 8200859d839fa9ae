"""Expert-parallel token exchange: the library manager on two and three gloo ranks against the single-process expert oracle."""
import os

import pytest
import torch
import torch.multiprocessing as mp


class _Experts:
    """The part of ``FusedMoE`` the managers use: this rank's slice of a seeded stack of experts."""

    def __init__(self, E, n, rank, H, I, dtype=torch.float32, device="cpu"):
        g = torch.Generator().manual_seed(1)
        w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.2).to(dtype)
        w2 = (torch.randn(E, H, I, generator=g) * 0.2).to(dtype)
        self.full = (w13, w2)
        self.E_local, self.e_off = E // n, rank * (E // n)
        self.w13 = w13[self.e_off:self.e_off + self.E_local].to(device)
        self.w2 = w2[self.e_off:self.e_off + self.E_local].to(device)
        self.kernel_state = None

    def dequantized(self):
        return self.w13, self.w2


def _batch(T, H, E, k, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g)
    logits = torch.randn(T, E, generator=g)
    w, ids = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    return x, w / w.sum(-1, keepdim=True), ids.to(torch.int32)


def _worker(rank, n, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=n)
    from onecat_vllm.ops import ref
    from onecat_vllm.parallel.all2all import TorchAll2All, token_slice
    E, k, H, I = 6 * n, 3, 32, 16
    layer = _Experts(E, n, rank, H, I)
    mgr = TorchAll2All(n, rank)
    ok, msgs = True, []
    for T in (1, 5, 16, 33):   # fewer tokens than ranks leaves some ranks with nothing to route: they take part all the same
        x, w, ids = _batch(T, H, E, k, seed=T)
        want = ref.fused_experts(x, layer.full[0], layer.full[1], w, ids.long())
        lo, hi = token_slice(T, n, rank)
        got = mgr.moe(layer, x[lo:hi], w[lo:hi], ids[lo:hi], t_off=lo, T_total=T, gather=True)
        err = (got - want).abs().max().item()
        if got.shape != want.shape or err > 1e-4:
            ok = False
            msgs.append(f"T={T} err={err}")
        local = mgr.moe(layer, x[lo:hi], w[lo:hi], ids[lo:hi])
        if hi > lo and (local - want[lo:hi]).abs().max().item() > 1e-4:
            ok = False
            msgs.append(f"T={T} local rows differ")
    q.put((rank, ok, msgs))
    dist.destroy_process_group()


@pytest.mark.timeout(180)
@pytest.mark.parametrize("n", [2, 3])
def test_torch_all2all_matches_single_process_experts(n):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + n
    procs = [ctx.Process(target=_worker, args=(r, n, port, q)) for r in range(n)]
    for p in procs:
        p.start()
    res = [q.get(timeout=150) for _ in range(n)]
    for p in procs:
        p.join(30)
    assert all(ok for _, ok, _ in res), res


def test_token_slice_covers_the_batch_once():
    from onecat_vllm.parallel.all2all import token_slice
    for T in (0, 1, 7, 64, 1025):
        for n in (2, 4, 8):
            cuts = [token_slice(T, n, r) for r in range(n)]
            assert cuts[0][0] == 0 and cuts[-1][1] == T and all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            assert max(hi - lo for lo, hi in cuts) - min(hi - lo for lo, hi in cuts) <= 1
