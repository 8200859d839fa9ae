"""Micro-benchmark of the tensor-parallel fused paths against NCCL, one process per GPU:

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m onecat_vllm.parallel.bench_comm [--json PATH]

For each token count T it times (CUDA events on the launching stream, max over ranks, median of ``--iters`` samples of ``--inner`` back-to-back calls each, after 5 warm-up rounds):
  * ``fused``  : peer-memory reduce + residual add + RMSNorm in one kernel (one-shot for small T: flag-free arrival buffers, or the
    flag handshake with ``ONECAT_TP_ONESHOT=flags``; reduce-scatter/all-gather two-shot above)
  * ``nccl``   : ncclAllReduce followed by the fused add+RMSNorm kernel (the baseline path)
  * ``gemm+fused`` / ``gemm+push+fused`` : a row-parallel bf16 GEMM (K = 17408 / N ranks → 5120) followed by the reduction, with the
    GEMM epilogue leaving its tile local (pulled by the reduction) or storing it straight into the peers' slabs.
Roofline: bytes that must cross NVLink per rank ÷ 770 GB/s (measured peer copy bandwidth per direction) and GEMM FLOPs ÷ measured
bf16 peak; the reported fraction is max(those two) ÷ measured time."""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--inner", type=int, default=20)
    ap.add_argument("--json", default="")
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--sizes", default="1,16,64,256,1024,8192")
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from onecat_vllm.ops import cuda as K
    from onecat_vllm.parallel.fused import LAMPORT, NVLS, ONE_SHOT, TWO_SHOT, FusedTP
    H = a.hidden
    f = FusedTP(world, rank, dev, 8192, H)
    w = torch.ones(H, device=dev, dtype=torch.bfloat16)
    Kin = 17408 // world // 64 * 64
    wg = (torch.randn(H, Kin, device=dev) * 0.02).bfloat16()
    rows = []

    def timed(fn):
        # `inner` back-to-back calls per sample: the ranks leave the barrier at slightly different times, and a single
        # call would mostly measure that skew (each rank waits for the slowest one inside the collective)
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        ts = []
        for _ in range(a.iters):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            dist.barrier()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(a.inner):
                fn()
            e1.record()
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / a.inner], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t))
        ts.sort()
        return ts[len(ts) // 2]

    sizes = [int(x) for x in a.sizes.split(",")]
    # with multicast support every size is measured twice: through the switch and with the peer-store kernels
    passes = [(T, nv) for T in sizes for nv in ((True, False) if f.nv is not None else (False,))]
    for T, use_nv in passes:
        f.nvls_mode = "always" if use_nv else "never"
        part = torch.randn(T, H, device=dev).bfloat16()
        res = torch.randn(T, H, device=dev).bfloat16()
        x = torch.randn(T, Kin, device=dev).bfloat16()
        mode = f.mode_for(T)

        def fused():
            if mode == LAMPORT:   # the flag-free kernel sends the rows itself from wherever they are: no staging copy to subtract
                f.reduce_add_norm(part, res, w, 1e-6, False)
                return
            buf = f.partial_buffer(T, H, torch.bfloat16)
            buf.copy_(part)
            f.reduce_add_norm(buf, res, w, 1e-6, False)

        def copy_only():
            f.partial_buffer(T, H, torch.bfloat16).copy_(part)

        def nccl():
            p2 = part.clone()
            dist.all_reduce(p2)
            K.rms_norm(p2, w, 1e-6, res, False)

        def clone_only():
            part.clone()

        def gemm_pull():
            buf = f.partial_buffer(T, H, torch.bfloat16)
            K.gemm_bf16(x, wg, out=buf)
            f.reduce_add_norm(buf, res, w, 1e-6, False)

        def gemm_push():
            if mode == NVLS:   # the switch pulls the partial sums: there is no push form
                return gemm_pull()
            buf = f.partial_buffer(T, H, torch.bfloat16)
            K._gemm(x, wg, None, None, buf, None, H, H, H, 0, 0, 1, push=f.push_spec(T))
            f.reduce_add_norm(buf, res, w, 1e-6, False, pushed=True)

        def gemm_nccl():
            y = K.gemm_bf16(x, wg)
            dist.all_reduce(y)
            K.rms_norm(y, w, 1e-6, res, False)

        # device time without the host's launch rate: `inner` reductions captured in one CUDA graph (the decode path replays graphs)
        t_graph = None
        if mode in (LAMPORT, NVLS):
            src = part if mode == LAMPORT else f.partial_buffer(T, H, torch.bfloat16)
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    f.reduce_add_norm(f.partial_buffer(T, H, torch.bfloat16) if mode == NVLS else part, res, w, 1e-6, False)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            dist.barrier()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for _ in range(a.inner):
                    f.reduce_add_norm(f.partial_buffer(T, H, torch.bfloat16) if mode == NVLS else part, res, w, 1e-6, False)
            keep, a.inner = a.inner, 1
            t_graph = timed(gr.replay) / keep
            a.inner = keep
            del src
        t_f, t_c = timed(fused), (0.0 if mode == LAMPORT else timed(copy_only))
        t_n, t_cl = timed(nccl), timed(clone_only)
        t_gp, t_gpush, t_gn = timed(gemm_pull), timed(gemm_push), timed(gemm_nccl)
        # bytes each rank must receive over NVLink for the reduction (+ send for the gather in two-shot mode)
        if mode in (ONE_SHOT, LAMPORT):
            link_bytes = (world - 1) * T * H * 2
        elif mode == NVLS:   # a rank receives the reduced rows it owns and everybody else's normalised and residual rows
            link_bytes = (1.0 / world + 2.0 * (world - 1) / world) * T * H * 2
        else:
            link_bytes = 2 * (world - 1) / world * T * H * 2
        t_link = link_bytes / 770e9 * 1e3
        t_flop = 2.0 * T * H * Kin / 1648e12 * 1e3
        rows.append(dict(T=T, switch=bool(use_nv), mode={ONE_SHOT: "one-shot (flags)", LAMPORT: "one-shot (flag-free)", TWO_SHOT: "two-shot", NVLS: "switch (multimem)"}[mode], fused_ms=t_f - t_c, fused_in_graph_ms=t_graph, nccl_plus_norm_ms=t_n - t_cl,
                         gemm_pull_fused_ms=t_gp, gemm_push_fused_ms=t_gpush, gemm_nccl_norm_ms=t_gn, link_bound_ms=t_link,
                         roofline_frac_reduce=t_link / max(t_f - t_c, 1e-9), roofline_frac_gemm_fused=max(t_link, t_flop) / min(t_gp, t_gpush)))
    st = K.check_status()
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
        print(json.dumps({"world": world, "device_status": st}))
        if a.json:
            json.dump({"world": world, "rows": rows, "device_status": st}, open(a.json, "w"), indent=1)
    dist.barrier()
    torch.cuda.synchronize()
    f.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
