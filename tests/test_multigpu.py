"""Real NCCL runs on two GPUs (skipped on a single-GPU box): the
sequence-sharded scan and the batch x channel sharded scan against the
one-shot scan on one GPU."""

import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, mode, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist

    import kla_b200
    from test_scan_gpu import INPUTS, _seeded

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        # "block1": one batch element, so the two ranks split the CHANNELS and dk, dq are all-reduced over NCCL
        B, L, M, S = (1 if mode == "block1" else 2), 96, 64, 16
        g = _seeded(B, L, M, S, seed=77)
        t = lambda n: torch.tensor(g[n], dtype=torch.float32, device=dev)
        full = [t(n).requires_grad_(True) for n in INPUTS]
        lam0, eta0 = t("lam0").requires_grad_(True), t("eta0").requires_grad_(True)
        dy, dyv, dl, de = t("dy"), t("dyvar"), t("dlam_fin"), t("deta_fin")
        # one-shot reference on this GPU
        y_ref, yv_ref, st_ref = kla_b200.kla_scan_b200(*full, initial_state=(lam0, eta0))
        loss = (y_ref * dy).sum() + (yv_ref * dyv).sum() + (st_ref.lam * dl).sum() + (st_ref.eta * de).sum()
        g_ref = torch.autograd.grad(loss, full + [lam0, eta0])
        v, lv, k, qq, a, p = full
        out = {}
        if mode == "seq":
            sl = slice(rank * L // world, (rank + 1) * L // world)
            y, yv, st = kla_b200.kla_scan_seq_sharded(v[:, sl], lv[:, sl], k[:, sl], qq[:, sl], a, p,
                                                      initial_state=(lam0, eta0))
            loss = (y * dy[:, sl]).sum() + (yv * dyv[:, sl]).sum()
            if rank == world - 1:
                loss = loss + (st.lam * dl).sum() + (st.eta * de).sum()
            gr = torch.autograd.grad(loss, full + [lam0, eta0])
            out["y"] = (y - y_ref[:, sl]).abs().max().item()
            out["lam"] = (st.lam - st_ref.lam).abs().max().item()
            names = ["dv", "dlv", "dk", "dq", "da", "dp", "dlam0", "deta0"]
            for n, a_, b_ in zip(names, gr, g_ref):
                if n in ("dv", "dlv", "dk", "dq"):
                    a_, b_ = a_[:, sl], b_[:, sl]
                out[n] = ((a_ - b_).abs().max() / (b_.abs().max() + 1)).item()
        else:
            sh = kla_b200.shard
            blk = sh.block_of(B, M, world, rank)
            groups = sh.make_groups(world, blk.batch_parts, blk.channel_parts)
            bv, blv, bk, bq, ba, bp, bst = sh.take_block(blk, v, lv, k, qq, a, p, (lam0, eta0))
            y, yv, st = sh.scan_block(kla_b200.kla_scan_b200, groups, bv, blv, bk, bq, ba, bp, initial_state=bst)
            bs, ms = slice(blk.b0, blk.b1), slice(blk.m0, blk.m1)
            loss = ((y * dy[bs, :, ms]).sum() + (yv * dyv[bs, :, ms]).sum()
                    + (st.lam * dl[bs, ms]).sum() + (st.eta * de[bs, ms]).sum())
            gr = torch.autograd.grad(loss, full + [lam0, eta0])
            out["y"] = (y - y_ref[bs, :, ms]).abs().max().item()
            out["dv"] = ((gr[0][bs, :, ms] - g_ref[0][bs, :, ms]).abs().max() / (g_ref[0].abs().max() + 1)).item()
            assert (blk.batch_parts, blk.channel_parts) == ((1, 2) if mode == "block1" else (2, 1))
            out["dk"] = ((gr[2][bs] - g_ref[2][bs]).abs().max() / (g_ref[2].abs().max() + 1)).item()
            out["dq"] = ((gr[3][bs] - g_ref[3][bs]).abs().max() / (g_ref[3].abs().max() + 1)).item()
            out["da"] = ((gr[4][ms] - g_ref[4][ms]).abs().max() / (g_ref[4].abs().max() + 1)).item()
            out["dp"] = ((gr[5][ms] - g_ref[5][ms]).abs().max() / (g_ref[5].abs().max() + 1)).item()
        torch.cuda.synchronize()
        q.put((rank, out))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["seq", "block", "block1"])
def test_two_gpu_sharding_matches_one_shot(mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 32500 + (os.getpid() % 2000) + ["seq", "block", "block1"].index(mode)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    [p.start() for p in procs]
    res = [q.get(timeout=300) for _ in procs]
    [p.join(timeout=60) for p in procs]
    assert all(p.exitcode == 0 for p in procs)
    for rank, out in res:
        print(rank, out)
        for n, e in out.items():
            assert e < 2e-4, f"rank {rank} {mode}: {n} {e:.2e}"
