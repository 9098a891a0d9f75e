#!/usr/bin/env python3
"""Benchmark of the quantized-inference hot path on B200 (one process per GPU).

Default workload (``--workload c2``): continuous-batching decode through the 7 affine 4-bit g64
projections of a Llama-3-8B-shaped layer (q,o 4096->4096; k,v 4096->1024; gate,up 4096->14336;
down 14336->4096) for M concurrent sequences per GPU.  A *step* is one pass of M token rows through
``--layers`` distinct layers' weight sets (distinct so the working set, ~123 MB per layer, is far
larger than the 126 MB L2 and every pass streams the weights from HBM).  The metric is decode
tokens/s through one such layer: value = n_gpus * M * layers * steps / time.  Sequences are
batch-sharded: every GPU holds a full weight replica and its own M rows; no communication.

Synthetic data: weights ~N(0,0.02) quantized on the device with the library's own quantize, activations
~N(0,1) bf16, seeded.  Every launch goes through the C ABI (libqb200.so) via ctypes; the timed region is
a CUDA graph of those launches replayed ``--steps`` times between CUDA events.

``--impl reference`` times the CPU restatement of the same path (oracle/, the stand-in for MLX's CPU
backend, which is not in the reference checkout) on the host cores for the same metric.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "mlx-serve_b200"))

LLAMA = [("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
         ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336)]
BITS, GS = 4, 64


def layer_bytes(M, bits=BITS, gs=GS):
    """Algorithmic bytes of one layer pass: packed weights + scales + biases + activations in + out."""
    tot = 0
    for _, n, k in LLAMA:
        tot += n * k * bits // 8 + 2 * (n * (k // gs) * 2) + M * k * 2 + M * n * 2
    return tot


# dram__bytes_read.sum + dram__bytes_write.sum over the algorithmic bytes of the same launches, from the ncu
# capture of one layer's launches: 14.29 + 9.57 + 66.71 + 33.33 MB measured for the four
# launches of a layer at M=8 (q/k/v, o, gate/up, down) against 124.0 MB algorithmic.  Traffic scales with the
# bytes a launch streams.
NCU_TRAFFIC_OVER_ALGORITHMIC = 123.90 / 123.99


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.idx = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                                  ("sw_power_cap", 8)):
                    if r[col].lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_layer_pass(M, seed=0xC2, reps=None, budget_s=12.0):
    """Oracle timing of one layer pass (7 projections) at M rows; returns (tokens/s, threads, sample text)."""
    import numpy as np
    from oracle import qoracle as qo
    # all the host threads this process may use (torchrun exports OMP_NUM_THREADS=1)
    try:
        qo.set_num_threads(len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        qo.set_num_threads(os.cpu_count() or 1)
    rng = np.random.default_rng(seed)
    ws, xs = [], {}
    for _, n, k in LLAMA:
        q = rng.integers(0, 2 ** 32, size=(n, k * BITS // 32), dtype=np.uint32)
        s = qo.f32_to_bf16((np.abs(rng.standard_normal((n, k // GS))) * 0.005 + 1e-3).astype(np.float32))
        b = qo.f32_to_bf16((rng.standard_normal((n, k // GS)) * 0.04).astype(np.float32))
        ws.append((q, s, b))
        if k not in xs:
            xs[k] = qo.bf16_round(rng.standard_normal((M, k)).astype(np.float32))

    def one():
        for (q, s, b), (_, n, k) in zip(ws, LLAMA):
            qo.qmm(xs[k], q, s, b, GS, BITS)

    one()  # warm
    t0 = time.perf_counter()
    one()
    dt1 = time.perf_counter() - t0
    n = reps if reps is not None else max(1, min(50, int(budget_s / max(dt1, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(n):
        one()
    dt = (time.perf_counter() - t0) / n
    return M / dt, qo.num_threads(), f"{n} passes of one layer (7 projections) at M={M}, weights of random codes", dt


def run_reference(args):
    """The reference arm: the CPU restatement of the path on the host cores, same metric."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    M = args.m
    steps, warmup = args.steps, args.warmup
    reps = max(1, warmup) + steps
    import numpy as np  # noqa: F401
    tps, threads, sample, dt = cpu_layer_pass(M, reps=None, budget_s=max(4.0, min(40.0, 2.0 * reps)))
    out = {
        "impl": "reference", "metric": "decode_tokens_per_s_llama3_8b_layer_q4g64", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "c2: Llama-3-8B layer, 7 projections, 4-bit g64, M=%d rows; CPU oracle port "
                               "(MLX CPU backend absent from the reference checkout)" % M, "M_per_gpu": M},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=8, help="concurrent sequences (token rows) per GPU")
    ap.add_argument("--layers", type=int, default=16, help="distinct layer weight sets rotated through per step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--sweep", action="store_true", help="also report M in {1,8,32,128} (outside the timed steps)")
    ap.add_argument("--no-batch", action="store_true", help="seven separate calls per layer instead of four")
    ap.add_argument("--micro-kv", action="store_true", help="decode attention over the packed KV cache (config 5) and exit")
    ap.add_argument("--micro-moe", action="store_true", help="routed-MoE gather_qmm decode (config 3, 64 tokens) and exit")
    ap.add_argument("--micro-moe-ep", action="store_true",
                    help="expert-parallel MoE block (config 3, 64 tokens per GPU) over all ranks and exit")
    ap.add_argument("--micro-prefill", action="store_true", help="dense prefill qmm (config 4) and exit")
    ap.add_argument("--micro", action="store_true", help="per-projection timings (us per launch, GB/s) and exit")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    import qb200

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    qb200.lib()  # fail loudly if the library is not built

    M, L = args.m, (0 if (args.micro_kv or args.micro_prefill or args.micro_moe or args.micro_moe_ep) else args.layers)
    g = torch.Generator(device=dev).manual_seed(0xC2 + rank)
    layers = []
    for _ in range(L):
        ws = []
        for _, n, k in LLAMA:
            w = (torch.randn((n, k), device=dev, generator=g) * 0.02).to(torch.bfloat16)
            ws.append(qb200.quantize(w, GS, BITS))
            del w
        layers.append(ws)

    def make_io(m):
        xin = torch.randn((L, m, 4096 + 14336), device=dev, generator=g).to(torch.bfloat16)
        nout = sum(n for _, n, _ in LLAMA)
        yout = torch.empty((L, m, nout), dtype=torch.bfloat16, device=dev)
        return xin, yout

    cols, c0 = [], 0
    for _, n, _ in LLAMA:
        cols.append((c0, c0 + n))
        c0 += n

    def enqueue(xin, yout):
        # 7 projections per layer in 4 calls: (q,k,v) and (gate,up) share their input, so they go through the
        # batch entry point (one launch each); o and down are single calls.
        for li in range(L):
            xh, xd = xin[li, :, :4096], xin[li, :, 4096:]
            out = [yout[li, :, a:b] for a, b in cols]
            if args.no_batch:
                for i, (name, n, k) in enumerate(LLAMA):
                    qb200.quantized_matmul(xd if k != 4096 else xh, *layers[li][i], True, GS, BITS, out=out[i])
                continue
            qb200.quantized_matmul_batch(xh, layers[li][0:3], out[0:3], True, GS, BITS)
            qb200.quantized_matmul(xh, *layers[li][3], True, GS, BITS, out=out[3])
            qb200.quantized_matmul_batch(xh, layers[li][4:6], out[4:6], True, GS, BITS)
            qb200.quantized_matmul(xd, *layers[li][6], True, GS, BITS, out=out[6])

    def build_graph(m):
        xin, yout = make_io(m)
        s = torch.cuda.Stream(device=dev)
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            enqueue(xin, yout)  # sets kernel attributes, warms up
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            enqueue(xin, yout)
        return gr, xin, yout

    def time_graph(gr, steps, warmup):
        for _ in range(warmup):
            gr.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms = float(t.item())
        return ms

    if args.micro_moe_ep:
        from qb200 import ep
        E, H, I, T, topk = 128, 2048, 768, 64, 8
        per = E // world
        banks = {}
        for name, (n, k) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
            w = (torch.randn((per, n, k), device=dev, generator=g) * 0.02).to(torch.bfloat16)
            banks[name] = qb200.quantize(w, 64, 4)
            del w
        fn = ep.default_expert_fn(banks)
        xtok = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
        inds, wts = ep.route(torch.randn((T, E), device=dev, generator=g), topk)
        res = {"n_gpus": world, "experts_per_gpu": per}
        for name, block in (("exact_counts", ep.moe_block_ep), ("padded_no_host_sync", ep.moe_block_ep_padded)):
            for _ in range(3):
                out = block(xtok, inds, wts, E, fn)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(args.steps):
                out = block(xtok, inds, wts, E, fn)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            if world > 1:
                tt = torch.tensor([ms], device=dev)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                ms = float(tt.item())
            res[name] = {"ms_per_block": ms, "tokens_per_s": world * T / (ms * 1e-3), "nan": bool(torch.isnan(out).any())}
        # (Both plans are timed eagerly.  Capturing the padded plan's collectives into a CUDA graph did not return on
        # a two-GPU box and is not attempted.)
        if rank == 0:
            print(json.dumps(res))
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    if args.micro_moe:
        E, H, I, T, topk = 128, 2048, 768, 64, 8
        banks = {}
        for name, (n, k) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
            w = (torch.randn((E, n, k), device=dev, generator=g) * 0.02).to(torch.bfloat16)
            banks[name] = qb200.quantize(w, 64, 4)
            del w
        per_expert = 786432 + 2 * 49152
        res = {}

        def block(T, inds, fused=False):
            """Buffers and the three gather_qmm calls of one MoE block for T tokens routed to `inds` [T*topk]."""
            order = torch.argsort(inds, stable=True)
            sorted_inds = inds[order].to(torch.int32).contiguous()
            xtok = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
            x_rep = xtok[order // topk].reshape(T * topk, 1, H).contiguous()
            act = torch.randn((T * topk, 1, I), device=dev, generator=g).to(torch.bfloat16)
            yg = torch.empty((T * topk, 1, I), dtype=torch.bfloat16, device=dev)
            yu = torch.empty_like(yg)
            yd = torch.empty((T * topk, 1, H), dtype=torch.bfloat16, device=dev)
            inv = torch.argsort(order).to(torch.int32).contiguous()
            scores = torch.softmax(torch.randn((T, topk), device=dev, generator=g), -1).to(torch.bfloat16)
            ysum = torch.empty((T, H), dtype=torch.bfloat16, device=dev)

            def run():
                if fused:   # gate and up in one launch with the SwiGLU epilogue, its result feeds the down projection
                    qb200.gather_qmm_swiglu(x_rep, *banks["gate"], *banks["up"], None, sorted_inds, 64, 4,
                                            sorted_indices=True, out=yg)
                    if T == 1:   # single-token decode step: down projection, weighting and sum over top-k in one launch
                        qb200.moe_down_reduce(yg.view(T, topk, I), *banks["down"], sorted_inds.view(T, topk), scores, 64, 4,
                                              out=ysum)
                        return
                    qb200.gather_qmm(yg, *banks["down"], None, sorted_inds, True, 64, 4, sorted_indices=True, out=yd)
                    qb200.moe_weighted_sum(yd, scores, inv, out=ysum)   # back to token order, x scores, sum over top-k
                    return
                qb200.gather_qmm(x_rep, *banks["gate"], None, sorted_inds, True, 64, 4, sorted_indices=True, out=yg)
                qb200.gather_qmm(x_rep, *banks["up"], None, sorted_inds, True, 64, 4, sorted_indices=True, out=yu)
                qb200.gather_qmm(act, *banks["down"], None, sorted_inds, True, 64, 4, sorted_indices=True, out=yd)
            return run, int(torch.unique(sorted_inds).numel())

        # 64 tokens: one block touches (nearly) every expert, 340 MB of banks > L2.  4096 tokens (prefill): 32768
        # routed rows, 256 per expert on average -- a grouped GEMM; reported in TFLOP/s as well.
        # 1 token: 16 blocks in the graph, each routed to a disjoint set of 8 experts, so the replay still
        # streams all 128 experts from HBM instead of re-reading 21 MB from L2.
        for T, fused in ((64, False), (1, False), (4096, False), (64, True), (1, True)):
            if T != 1:
                logits = torch.randn((T, E), device=dev, generator=g)
                runs = [block(T, torch.topk(torch.softmax(logits, -1), topk, dim=-1).indices.reshape(-1), fused)]
            else:
                perm = torch.randperm(E, device=dev, generator=g)
                runs = [block(T, perm[i * topk:(i + 1) * topk], fused) for i in range(E // topk)]
            for r, _ in runs:
                r()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for r, _ in runs:
                    r()
            ms = time_graph(gr, args.steps, 3) / args.steps / len(runs)
            uniq = runs[0][1]
            by = 3 * uniq * per_expert + T * topk * 2 * (2 * (H + I) + (I + H))
            res[f"tokens{T}" + ("_fused_block" if fused else "")] = {"us_per_block": ms * 1e3, "unique_experts": uniq, "bytes": by,
                                 "GBps": by / (ms * 1e-3) / 1e9,
                                 "TFLOPs": 2.0 * T * topk * 3 * H * I / (ms * 1e-3) / 1e12}
            del gr
        if rank == 0:
            print(json.dumps(res))
        return

    if args.micro_prefill:
        res = {}
        Mp, Np, Kp = 2048, 14336, 4096
        x = torch.randn((Mp, Kp), device=dev, generator=g).to(torch.bfloat16)
        for bits in (4, 8):
            ws = []
            for _ in range(4):  # rotate weight sets (4 x 33-62 MB) and outputs
                w = (torch.randn((Np, Kp), device=dev, generator=g) * 0.02).to(torch.bfloat16)
                ws.append(qb200.quantize(w, 64, bits))
                del w
            y = torch.empty((4, Mp, Np), dtype=torch.bfloat16, device=dev)

            def run():
                for i in range(4):
                    qb200.quantized_matmul(x, *ws[i], True, 64, bits, out=y[i])
            run()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                run()
            ms = time_graph(gr, args.steps, 3) / args.steps / 4
            res[f"b{bits}"] = {"ms_per_call": ms, "TFLOPs": 2.0 * Mp * Np * Kp / (ms * 1e-3) / 1e12,
                               "tc_status": qb200.lib().qb200_debug_tc_status()}
            del ws, y
        if rank == 0:
            print(json.dumps(res))
        return

    if args.micro_kv:
        res = {}
        B, Hq, Hkv, D = 16, 32, 8, 128
        for T in (4096, 32768):
            for bits in (4, 8):
                ncache = 4 if T == 4096 else 1   # rotate caches so every call streams from HBM (126 MB L2)
                cap = T + 256                    # views of a larger capacity buffer: head stride != T * last
                caches = []
                for _ in range(ncache):
                    k = torch.randn((B, Hkv, cap, D), device=dev, generator=g).to(torch.bfloat16)
                    kt = qb200.quantize(k, 64, bits)
                    k.normal_(generator=g)
                    vt = qb200.quantize(k, 64, bits)
                    del k
                    caches.append(([t_[:, :, :T] for t_ in kt], [t_[:, :, :T] for t_ in vt]))
                q = torch.randn((B, Hq, 1, D), device=dev, generator=g).to(torch.bfloat16)
                out = torch.empty_like(q)
                ws = torch.empty(qb200.kv_decode_attention_workspace_size(B, Hq, Hkv, T, D), dtype=torch.uint8, device=dev)
                reps = 8

                def run():
                    for i in range(reps):
                        kt, vt = caches[i % ncache]
                        qb200.kv_decode_attention(q, kt, vt, bits, 64, D ** -0.5, workspace=ws, out=out)
                run()
                torch.cuda.synchronize()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    run()
                ms = time_graph(gr, args.steps, 3) / args.steps / reps
                by = B * Hkv * T * 2 * (D * bits // 8 + 8) + 2 * B * Hq * D * 2
                res[f"T{T}_b{bits}"] = {"us_per_call": ms * 1e3, "GBps": by / (ms * 1e-3) / 1e9, "bytes": by}
                del caches
        if rank == 0:
            print(json.dumps(res))
        return

    if args.micro:
        res = {}
        for m in (1, 8):
            for name, n, k in [LLAMA[0], LLAMA[1], LLAMA[4], LLAMA[6]]:
                idx = [i for i, (nm, _, _) in enumerate(LLAMA) if nm == name][0]
                x = torch.randn((m, k), device=dev, generator=g).to(torch.bfloat16)
                y = torch.empty((L, m, n), dtype=torch.bfloat16, device=dev)

                def run():
                    for li in range(L):
                        q, s, b = layers[li][idx]
                        qb200.quantized_matmul(x, q, s, b, True, GS, BITS, out=y[li])
                run()
                torch.cuda.synchronize()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr):
                    run()
                ms = time_graph(gr, args.steps, 3) / args.steps
                by = n * k * BITS // 8 + 4 * n * (k // GS) + 2 * m * (n + k)
                res[f"{name}_M{m}"] = {"us_per_launch": ms * 1e3 / L, "GBps": by * L / (ms * 1e-3) / 1e9}
        if rank == 0:
            print(json.dumps(res))
        return

    gr, xin, yout = build_graph(M)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms = time_graph(gr, args.steps, max(args.warmup, 3))
    ms_step = ms / args.steps
    value = world * M * L * args.steps / (ms * 1e-3)

    # end to end: host buffers in, host buffers out, copies inside the timed region.  Every step copies its inputs
    # from pinned host memory and its outputs back; two sets of device buffers (two graphs over the same weights)
    # alternate, so that the copies of one step overlap the kernels of its neighbours, as a serving loop would run it.
    gr2, xin2, yout2 = build_graph(M)
    sets = [(gr, xin, yout), (gr2, xin2, yout2)]
    xin_h = [torch.empty(xin.shape, dtype=xin.dtype, pin_memory=True).copy_(xin) for _ in range(2)]
    yout_h = [torch.empty(yout.shape, dtype=yout.dtype, pin_memory=True) for _ in range(2)]
    s_main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

    def e2e_steps(n):
        ev_in = [None, None]; ev_comp = [None, None]; ev_out = [None, None]
        for i in range(n):
            b = i & 1
            g_b, x_b, y_b = sets[b]
            with torch.cuda.stream(s_in):
                if ev_comp[b] is not None:
                    s_in.wait_event(ev_comp[b])        # the kernels that read this input buffer two steps ago
                x_b.copy_(xin_h[b], non_blocking=True)
                ev_in[b] = torch.cuda.Event(); ev_in[b].record(s_in)
            s_main.wait_event(ev_in[b])
            if ev_out[b] is not None:
                s_main.wait_event(ev_out[b])           # the read-back of this output buffer two steps ago
            g_b.replay()
            ev_comp[b] = torch.cuda.Event(); ev_comp[b].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_comp[b])
                yout_h[b].copy_(y_b, non_blocking=True)
                ev_out[b] = torch.cuda.Event(); ev_out[b].record(s_out)
        s_main.wait_stream(s_in)
        s_main.wait_stream(s_out)

    s_in.wait_stream(s_main); s_out.wait_stream(s_main)
    e2e_steps(4)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_steps(args.steps)
    e1.record()
    torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    e2e_value = world * M * L * args.steps / (ms_e2e * 1e-3)

    # The single-token line of the same workload (the shape the bandwidth target is stated for) is cheap
    # and always reported next to the batch-decode headline.
    qmv_m1 = None
    if M != 1 and L > 0:
        g1, _, _ = build_graph(1)
        ms1 = time_graph(g1, args.steps, 3) / args.steps
        qmv_m1 = {"ms_per_step": ms1, "tokens_per_s": world * L / (ms1 * 1e-3), "hbm_gbs": L * layer_bytes(1) / (ms1 * 1e-3) / 1e9}
        del g1

    sweep = None
    if args.sweep:
        sweep = {}
        for m in (1, 8, 16, 32, 64, 128):
            g2, _, _ = build_graph(m)
            msw = time_graph(g2, args.steps, 3) / args.steps
            sweep[str(m)] = {"ms_per_step": msw, "tokens_per_s": world * m * L / (msw * 1e-3),
                             "hbm_gbs": L * layer_bytes(m) / (msw * 1e-3) / 1e9}
            del g2

    if rank == 0:
        peak, which = peaks()
        # the streaming kernel serves 8 tokens per launch (fused q/k/v and gate/up: 4 launches per layer); above
        # 32 tokens the tensor-core kernel takes one launch per projection
        launches_per_layer = 7 if M > 32 else (7 if args.no_batch else 4) * ((M + 7) // 8)
        achieved = L * layer_bytes(M) / (ms_step * 1e-3) / 1e9
        out = {
            "metric": "decode_tokens_per_s_llama3_8b_layer_q4g64", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "c2: continuous-batching decode through the 7 affine 4-bit g64 projections of a "
                                   "Llama-3-8B-shaped layer", "M_per_gpu": M, "layers_per_step": L,
                       "weights_bytes_per_step": L * (layer_bytes(0)), "l2": "inputs larger than L2 (%.0f MB of "
                       "weights streamed per step)" % (L * layer_bytes(0) / 1e6), "parallelism": "batch-sharded x%d, "
                       "weights replicated, no collective" % world},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": which, "frac_of_nominal_8TBs": achieved / 8000.0,
                         "bytes_per_launch": layer_bytes(M) / (7.0 if args.no_batch else 4.0), "kernel": "qmv_stream_kernel",
                         "traffic": NCU_TRAFFIC_OVER_ALGORITHMIC * layer_bytes(M) / (7.0 if args.no_batch else 4.0),
                         "traffic_source": "ncu dram__bytes_read+write of the four launches of one layer (2-layer "
                                           "capture), scaled by algorithmic bytes to the average launch"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": xin.numel() * 2,
                    "d2h_bytes_per_step": yout.numel() * 2, "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": args.steps * L * launches_per_layer,
            "clocks": clocks,
        }
        if qmv_m1:
            qmv_m1["frac_of_peak"] = qmv_m1["hbm_gbs"] / peak
            out["qmv_m1"] = qmv_m1
        if sweep:
            out["sweep_M"] = sweep
        if not args.no_cpu_baseline:
            tps, threads, sample, _ = cpu_layer_pass(M)
            out["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample}
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
