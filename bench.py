#!/usr/bin/env python3
"""Benchmark of the quantized-inference hot path on B200 (one process per GPU).

Headline workload (benchmark configuration 2): continuous-batching decode through the 7 affine 4-bit g64
projections of a Llama-3-8B-shaped layer (q,o 4096->4096; k,v 4096->1024; gate,up 4096->14336; down 14336->4096)
for M = 8 concurrent sequences per GPU.  One *pass* sends the M token rows through 16 distinct layers' weight sets
(distinct so that the working set, ~123 MB per layer, is far larger than the 126 MB L2 and every pass streams the
weights from HBM); a *step* is ``--repeats`` passes (128 by default), so that ``--steps 20`` times a region of about
two seconds.  The metric is decode token rows per second through one such layer:
value = n_gpus * M * 16 * repeats * steps / time.  (A token crosses 32 such layers in the full model:
``tokens_per_s_through_32_layers`` = value / 32.)  Sequences are batch-sharded: every GPU holds a full weight replica
and its own M rows; no communication.

Every launch goes through the C ABI (libqb200.so) via ctypes; a pass is one CUDA graph of those launches.  The same
JSON line carries, under ``configs``, the other benchmark configurations measured in the same run (C1 single qmv over
rotated weight sets, the C2 sweep over M, C3 routed-expert decode / prefill blocks, C4 dense prefill, C5 decode
attention over the packed KV cache), each with its fraction of the measured roofline.

Synthetic data: weights ~N(0,0.02) quantized on the device with the library's own quantize, activations ~N(0,1)
bf16, seeded.  ``--impl reference`` times the CPU restatement of the same path (oracle/, the stand-in for MLX's CPU
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
METRIC = "decode_tokens_per_s_llama3_8b_layer_q4g64"
# identical in both arms, so that their lines compare
CONFIG = {"workload": "c2: continuous-batching decode through the 7 affine 4-bit g64 projections of a Llama-3-8B-shaped "
                      "layer (q,o 4096->4096; k,v 4096->1024; gate,up 4096->14336; down 14336->4096)",
          "M_per_gpu": 8, "bits": BITS, "group_size": GS,
          "l2": "GPU arm: inputs larger than L2 (16 distinct layers = 1963 MB of weights streamed per pass)"}


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
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


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
        sm, mx, pw, reasons = [], None, [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
                pw.append(float(r[3]))
                for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                                  ("sw_power_cap", 8)):
                    if r[col].lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(pw) if pw else None}


class CpuLayer:
    """The oracle's pass of one layer (7 projections) at M rows, for the CPU baseline and the reference arm."""

    def __init__(self, M, seed=0xC2):
        import numpy as np
        from oracle import qoracle as qo
        self.qo, self.M = qo, M
        # all the host threads this process may use (torchrun exports OMP_NUM_THREADS=1)
        try:
            qo.set_num_threads(len(os.sched_getaffinity(0)))
        except (AttributeError, OSError):
            qo.set_num_threads(os.cpu_count() or 1)
        rng = np.random.default_rng(seed)
        self.ws, self.xs = [], {}
        for _, n, k in LLAMA:
            q = rng.integers(0, 2 ** 32, size=(n, k * BITS // 32), dtype=np.uint32)
            s = qo.f32_to_bf16((np.abs(rng.standard_normal((n, k // GS))) * 0.005 + 1e-3).astype(np.float32))
            b = qo.f32_to_bf16((rng.standard_normal((n, k // GS)) * 0.04).astype(np.float32))
            self.ws.append((q, s, b))
            if k not in self.xs:
                self.xs[k] = qo.bf16_round(rng.standard_normal((M, k)).astype(np.float32))

    def one_pass(self):
        for (q, s, b), (_, n, k) in zip(self.ws, LLAMA):
            self.qo.qmm(self.xs[k], q, s, b, GS, BITS)

    def time_passes(self, n):
        t0 = time.perf_counter()
        for _ in range(n):
            self.one_pass()
        return (time.perf_counter() - t0) / n


def run_reference(args):
    """The reference arm: the CPU restatement of the path on the host cores, same metric; a step is one pass of one
    layer (a bounded sample of the GPU arm's step), ``--warmup`` untimed passes then exactly ``--steps`` timed ones."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    M = args.m
    cpu = CpuLayer(M)
    for _ in range(max(1, args.warmup)):
        cpu.one_pass()
    dt = cpu.time_passes(args.steps)
    tps = M / dt
    sample = f"{args.steps} timed passes of one layer (7 projections) at M={M} after {max(1, args.warmup)} warm-up passes, weights of random codes"
    out = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(CONFIG, M_per_gpu=M),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cpu.qo.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "CPU oracle port (MLX's CPU backend is absent from the reference checkout); one step = one layer pass",
    }
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--m", type=int, default=8, help="concurrent sequences (token rows) per GPU")
    ap.add_argument("--layers", type=int, default=16, help="distinct layer weight sets per pass")
    ap.add_argument("--repeats", type=int, default=128, help="passes (graph replays) per step")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the other benchmark configurations (C1, C3, C4, C5, sweep)")
    ap.add_argument("--no-batch", action="store_true", help="seven separate calls per layer instead of four")
    ap.add_argument("--only", default="", help="comma list of c1,sweep,tick,c3,c4,c5,a7,qk,ep: run just these extra configurations and exit")
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
    hbm_peak, tc_peak, peak_src = peaks()
    only = [s for s in args.only.split(",") if s]

    M, L, R = args.m, args.layers, max(1, args.repeats)
    g = torch.Generator(device=dev).manual_seed(0xC2 + rank)

    def time_graph(gr, reps, warmup=3, sync_ranks=True):
        """Device time of `reps` replays (CUDA events on the launching stream), max over ranks."""
        for _ in range(warmup):
            gr.replay()
        torch.cuda.synchronize()
        if world > 1 and sync_ranks:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if world > 1 and sync_ranks:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
            ms = float(t.item())
        return ms

    def capture(fn):
        fn()   # sets kernel attributes, warms up
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            fn()
        return gr

    # ------------------------------------------------------------------ C2 weights and graphs
    layers = []
    if not only or "sweep" in only or "c1" in only or "tick" in only:
        for _ in range(L):
            ws = []
            for _, n, k in LLAMA:
                w = (torch.randn((n, k), device=dev, generator=g) * 0.02).to(torch.bfloat16)
                ws.append(qb200.quantize(w, GS, BITS))
                del w
            layers.append(ws)
    cols, c0 = [], 0
    for _, n, _ in LLAMA:
        cols.append((c0, c0 + n))
        c0 += n

    def make_io(m):
        xin = torch.randn((L, m, 4096 + 14336), device=dev, generator=g).to(torch.bfloat16)
        yout = torch.empty((L, m, c0), dtype=torch.bfloat16, device=dev)
        return xin, yout

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
        return capture(lambda: enqueue(xin, yout)), xin, yout

    def launches_per_layer(m):
        calls = 7 if args.no_batch else 4
        if m <= 8:
            return calls                      # the narrow streaming kernel, one launch per call
        if m <= 64:
            return 2 * calls                  # the wide streaming kernel and its activation pre-arrangement
        return 7                              # the tensor-core kernel, one launch per projection

    # ------------------------------------------------------------------ the other configurations
    def cfg_c1():
        """C1: one 4-bit qmv 1x4096 -> 4096, rotated over 64 distinct weight triples (604 MB >> L2) inside one graph."""
        nset = 64
        ws = []
        for _ in range(nset):
            w = (torch.randn((4096, 4096), device=dev, generator=g) * 0.02).to(torch.bfloat16)
            ws.append(qb200.quantize(w, GS, BITS))
            del w
        x = torch.randn((1, 4096), device=dev, generator=g).to(torch.bfloat16)
        y = torch.empty((nset, 1, 4096), dtype=torch.bfloat16, device=dev)

        def run():
            for i in range(nset):
                qb200.quantized_matmul(x, *ws[i], True, GS, BITS, out=y[i])
        gr = capture(run)
        ms = time_graph(gr, 40, sync_ranks=False) / 40 / nset
        by = 9453568
        return {"us_per_call": ms * 1e3, "bytes_per_call": by, "GBps": by / (ms * 1e-3) / 1e9,
                "frac_of_hbm_peak": by / (ms * 1e-3) / 1e9 / hbm_peak, "weight_sets_rotated": nset}

    def cfg_sweep():
        out = {}
        for m in (1, 16, 32, 64, 128):
            gr, _, _ = build_graph(m)
            ms = time_graph(gr, 20, sync_ranks=False) / 20
            gbs = L * layer_bytes(m) / (ms * 1e-3) / 1e9
            tfl = 2.0 * m * 218103808 * L / (ms * 1e-3) / 1e12
            out[f"M{m}"] = {"us_per_layer": ms * 1e3 / L, "tokens_per_s": m * L / (ms * 1e-3), "GBps": gbs,
                            "frac_of_hbm_peak": gbs / hbm_peak, "TFLOPs": tfl, "frac_of_bf16_peak": tfl / tc_peak}
            del gr
        return out

    def cfg_c3():
        """C3: routed-expert block, 128 experts top-8, hidden 2048, expert width 768, 4-bit g64: 64 tokens (decode),
        one token, 4096 tokens (prefill); router, device sort, gate/up (+SwiGLU), down, weighted sum all through the C ABI."""
        E, H, I, topk = 128, 2048, 768, 8
        banks = {}
        for name, (n, k) in (("gate", (I, H)), ("up", (I, H)), ("down", (H, I))):
            w = (torch.randn((E, n, k), device=dev, generator=g) * 0.02).to(torch.bfloat16)
            banks[name] = qb200.quantize(w, 64, 4)
            del w
        per_expert = 786432 + 2 * 49152
        res = {}

        def block(T, inds, fused):
            """Buffers and calls of one block for T tokens routed to `inds` [T, topk] (int32, on the device)."""
            xtok = torch.randn((T, H), device=dev, generator=g).to(torch.bfloat16)
            order, inv, sinds, rows, offs = qb200.moe_sort_by_expert(inds, E)
            x_rep = xtok[rows.long()].reshape(T * topk, 1, H).contiguous()
            yg = torch.empty((T * topk, 1, I), dtype=torch.bfloat16, device=dev)
            yu = torch.empty_like(yg)
            yd = torch.empty((T * topk, 1, H), dtype=torch.bfloat16, device=dev)
            scores = torch.softmax(torch.randn((T, topk), device=dev, generator=g), -1).to(torch.bfloat16)
            ysum = torch.empty((T, H), dtype=torch.bfloat16, device=dev)
            act = torch.randn((T * topk, 1, I), device=dev, generator=g).to(torch.bfloat16)

            def run():
                if fused:   # gate and up in one launch with the SwiGLU epilogue, its result feeds the down projection
                    qb200.gather_qmm_swiglu(x_rep, *banks["gate"], *banks["up"], None, sinds, 64, 4, sorted_indices=True, out=yg)
                    if T == 1:   # single-token decode step: down projection, weighting and sum over top-k in one launch
                        qb200.moe_down_reduce(yg.view(T, topk, I), *banks["down"], sinds.view(T, topk), scores, 64, 4, out=ysum)
                        return
                    qb200.gather_qmm(yg, *banks["down"], None, sinds, True, 64, 4, sorted_indices=True, out=yd)
                    qb200.moe_weighted_sum(yd, scores, inv, out=ysum)
                    return
                qb200.gather_qmm(x_rep, *banks["gate"], None, sinds, True, 64, 4, sorted_indices=True, out=yg)
                qb200.gather_qmm(x_rep, *banks["up"], None, sinds, True, 64, 4, sorted_indices=True, out=yu)
                qb200.gather_qmm(act, *banks["down"], None, sinds, True, 64, 4, sorted_indices=True, out=yd)
            return run, int(torch.unique(sinds).numel())

        for T, fused, label in ((64, True, "decode_64_tokens_fused_block"), (1, True, "decode_1_token_fused_block"),
                                (64, False, "decode_64_tokens_three_gather_qmm"), (4096, False, "prefill_4096_tokens_three_gather_qmm")):
            if T != 1:
                logits = torch.randn((T, E), device=dev, generator=g)
                runs = [block(T, qb200.moe_route(logits, topk)[0], fused)]
            else:   # 16 single-token blocks on disjoint expert sets: the replay streams all 128 experts from HBM
                perm = torch.randperm(E, device=dev, generator=g).to(torch.int32)
                runs = [block(T, perm[i * topk:(i + 1) * topk].reshape(1, topk).contiguous(), fused) for i in range(E // topk)]

            def run_all():
                for r, _ in runs:
                    r()
            gr = capture(run_all)
            ms = time_graph(gr, 20, sync_ranks=False) / 20 / len(runs)
            uniq = runs[0][1]
            by = 3 * uniq * per_expert + T * topk * 2 * (2 * (H + I) + (I + H))
            tfl = 2.0 * T * topk * 3 * H * I / (ms * 1e-3) / 1e12
            res[label] = {"us_per_block": ms * 1e3, "unique_experts": uniq, "bytes": by, "GBps": by / (ms * 1e-3) / 1e9,
                          "frac_of_hbm_peak": by / (ms * 1e-3) / 1e9 / hbm_peak, "TFLOPs": tfl,
                          "frac_of_bf16_peak": tfl / tc_peak, "tokens_per_s": T / (ms * 1e-3)}
            del gr
        # the device sort on its own (one launch): 64 x 8 and 4096 x 8 entries
        for T in (64, 4096):
            inds = qb200.moe_route(torch.randn((T, E), device=dev, generator=g), topk)[0]
            gr = capture(lambda: qb200.moe_sort_by_expert(inds, E))
            res[f"sort_by_expert_{T}_tokens_us"] = time_graph(gr, 50, sync_ranks=False) / 50 * 1e3
            del gr
        return res

    def cfg_c4():
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
            gr = capture(run)
            ms = time_graph(gr, 20, sync_ranks=False) / 20 / 4
            tfl = 2.0 * Mp * Np * Kp / (ms * 1e-3) / 1e12
            res[f"{bits}bit"] = {"ms_per_call": ms, "TFLOPs": tfl, "frac_of_bf16_peak": tfl / tc_peak,
                                 "status": qb200.lib().qb200_debug_tc_status()}
            del ws, y, gr
        return res

    def cfg_c5(seqs, shard_note):
        """C5: decode attention over the packed cache, Hq 32, Hkv 8, D 128, `seqs` sequences on this GPU."""
        res = {}
        Hq, Hkv, D = 32, 8, 128
        for T in (4096, 32768):
            for bits in (4, 8):
                ncache = 4 if T == 4096 else 1   # rotate caches so every call streams from HBM (126 MB L2)
                cap = T + 256                    # views of a larger capacity buffer: head stride != T * last
                caches = []
                for _ in range(ncache):
                    k = torch.randn((seqs, Hkv, cap, D), device=dev, generator=g).to(torch.bfloat16)
                    kt = qb200.quantize(k, 64, bits)
                    k.normal_(generator=g)
                    vt = qb200.quantize(k, 64, bits)
                    del k
                    caches.append(([t_[:, :, :T] for t_ in kt], [t_[:, :, :T] for t_ in vt]))
                q = torch.randn((seqs, Hq, 1, D), device=dev, generator=g).to(torch.bfloat16)
                out = torch.empty_like(q)
                ws = torch.empty(qb200.kv_decode_attention_workspace_size(seqs, Hq, Hkv, T, D), dtype=torch.uint8, device=dev)
                reps = 8

                def run():
                    for i in range(reps):
                        kt, vt = caches[i % ncache]
                        qb200.kv_decode_attention(q, kt, vt, bits, 64, D ** -0.5, workspace=ws, out=out)
                gr = capture(run)
                ms = time_graph(gr, 20, sync_ranks=world > 1 and seqs != 16) / 20 / reps
                by = seqs * Hkv * T * 2 * (D * bits // 8 + 8) + 2 * seqs * Hq * D * 2
                res[f"T{T}_{bits}bit"] = {"us_per_call": ms * 1e3, "bytes": by, "GBps_per_gpu": by / (ms * 1e-3) / 1e9,
                                          "frac_of_hbm_peak": by / (ms * 1e-3) / 1e9 / hbm_peak,
                                          "sequences_per_s_all_gpus": (world if seqs != 16 else 1) * seqs / (ms * 1e-3)}
                del caches, gr
        res["sharding"] = shard_note
        return res

    def cfg_attn_products(transpose):
        """The two products of the composed quantized attention as standalone operators, 16 sequences x 8 kv heads, GQA 4,
        D = 128: q @ K^T (transpose_w=true: queries [16, 8, 4, 128] with the packed key cache [16, 8, T, 128]) and
        attn @ V (transpose_w=false: probabilities [16, 8, 4, T] with the packed value cache)."""
        res = {}
        seqs, Hkv, gq, D = 16, 8, 4, 128
        for T in (4096, 4099, 32768):      # 4099: a cache length that rules vector loads of the probabilities out
            for bits in (4, 8):
                ncache = 8 if T < 32768 else 1   # rotate caches so every call streams from HBM (126 MB L2)
                caches = []
                for _ in range(ncache):
                    v = torch.randn((seqs, Hkv, T, D), device=dev, generator=g).to(torch.bfloat16)
                    caches.append(qb200.quantize(v, 64, bits))
                    del v
                if transpose:
                    xin = torch.randn((seqs, Hkv, gq, D), device=dev, generator=g).to(torch.bfloat16)
                    out = torch.empty((seqs, Hkv, gq, T), dtype=torch.bfloat16, device=dev)
                else:
                    xin = torch.softmax(torch.randn((seqs, Hkv, gq, T), device=dev, generator=g), dim=-1).to(torch.bfloat16)
                    out = torch.empty((seqs, Hkv, gq, D), dtype=torch.bfloat16, device=dev)
                reps = 8

                def run():
                    for i in range(reps):
                        qb200.quantized_matmul(xin, *caches[i % ncache], transpose, 64, bits, out=out)
                gr = capture(run)
                ms = time_graph(gr, 20, sync_ranks=False) / 20 / reps
                by = seqs * Hkv * T * (D * bits // 8 + (D // 64) * 4) + seqs * Hkv * gq * (T + D) * 2
                res[f"T{T}_{bits}bit"] = {"us_per_call": ms * 1e3, "bytes": by, "GBps": by / (ms * 1e-3) / 1e9,
                                          "frac_of_hbm_peak": by / (ms * 1e-3) / 1e9 / hbm_peak}
                del caches, gr
        return res

    def cfg_tick():
        """A whole decode tick of one Llama-3-8B-shaped layer through the library (forwardBatchedDecode's layer body,
        src/transformer.zig:9656-9861): q/k/v, rope + cache append, attention over per-sequence 4-bit caches (one launch: the splits of a
        sequence merge inside a thread-block cluster), o, add + norm, gate/up, SwiGLU, down, add + the next layer's input
        norm -- 10 launches (plus one norm before the
        first layer).  8 layers' weights rotate so the weights stream from HBM."""
        Hd, Hq, Hkv, D, F, NL = 4096, 32, 8, 128, 14336, 8
        lw = layers[:NL] if len(layers) >= NL else None
        if lw is None:
            return {"error": "needs the C2 layer weights"}
        res = {}
        wn = (1.0 + 0.1 * torch.randn((Hd,), device=dev, generator=g)).to(torch.bfloat16)
        for N, T in ((8, 4096), (16, 4096), (32, 1024)):
            cap = T + 256
            kt, vt = [], []
            for n in range(N):      # every sequence owns its cache (one set shared by the 8 layers of the replay)
                k = torch.randn((1, Hkv, cap, D), device=dev, generator=g).to(torch.bfloat16)
                kt.append(qb200.quantize(k, 64, 4))
                k.normal_(generator=g)
                vt.append(qb200.quantize(k, 64, 4))
                del k
            lens = [T - 1 - 7 * n for n in range(N)]
            kviews = [[t_[:, :, :lens[n] + 1] for t_ in kt[n]] for n in range(N)]
            vviews = [[t_[:, :, :lens[n] + 1] for t_ in vt[n]] for n in range(N)]
            offs = torch.tensor(lens, dtype=torch.int32, device=dev)
            h = torch.randn((N, Hd), device=dev, generator=g).to(torch.bfloat16)
            qkv = torch.empty((N, (Hq + 2 * Hkv) * D), dtype=torch.bfloat16, device=dev)
            outs = [qkv[:, :Hq * D], qkv[:, Hq * D:(Hq + Hkv) * D], qkv[:, (Hq + Hkv) * D:]]
            qk = qkv[:, :(Hq + Hkv) * D].view(N, Hq + Hkv, 1, D)
            q4, k4, v4 = outs[0].view(N, Hq, 1, D), outs[1].view(N, Hkv, 1, D), outs[2].view(N, Hkv, 1, D)
            attn = torch.empty((N, Hq, 1, D), dtype=torch.bfloat16, device=dev)
            ws = torch.empty(int(qb200.lib().qb200_kv_decode_attention_ptrs_workspace_size(N, Hq, Hkv, T, D)), dtype=torch.uint8, device=dev)
            bufs = {k_: torch.empty((N, n_), dtype=torch.bfloat16, device=dev) for k_, n_ in (("n1", Hd), ("o", Hd), ("h1", Hd), ("ff", Hd), ("g", F), ("u", F), ("act", F), ("d", Hd), ("h2", Hd))}

            def tick():
                hcur = h
                qb200.rms_norm(hcur, wn, 1e-5, out=bufs["n1"])          # the first layer's input norm
                for li in range(NL):
                    wq, wk, wv, wo, wg, wu, wd = lw[li]
                    qb200.quantized_matmul_batch(bufs["n1"], [wq, wk, wv], outs, True, GS, BITS)
                    qb200.kv_append_seqs(kt, vt, k4, v4, lens, 4, 64, rope_q=q4, rope_dims=D, rope_base=500000.0)   # + rope of q and k
                    qb200.kv_decode_attention_ptrs(q4, kviews, vviews, 4, 64, D ** -0.5, workspace=ws, out=attn)
                    qb200.quantized_matmul(attn.view(N, Hq * D), *wo, True, GS, BITS, out=bufs["o"])
                    qb200.add_rms_norm(hcur, bufs["o"], wn, 1e-5, sum_out=bufs["h1"], norm_out=bufs["ff"])
                    qb200.quantized_matmul_batch(bufs["ff"], [wg, wu], [bufs["g"], bufs["u"]], True, GS, BITS)
                    qb200.swiglu(bufs["g"], bufs["u"], out=bufs["act"])
                    qb200.quantized_matmul(bufs["act"], *wd, True, GS, BITS, out=bufs["d"])
                    # the residual add, fused with the next layer's input norm (the last layer: the add alone)
                    if li + 1 < NL:
                        qb200.add_rms_norm(bufs["h1"], bufs["d"], wn, 1e-5, sum_out=bufs["h2"], norm_out=bufs["n1"])
                    else:
                        qb200.add_rms_norm(bufs["h1"], bufs["d"], want_norm=False, sum_out=bufs["h2"])
                    hcur = bufs["h2"]
            gr = capture(tick)
            ms = time_graph(gr, 20, sync_ranks=False) / 20 / NL
            kv_bytes = sum(2 * Hkv * (lens[n] + 1) * (D * 4 // 8 + 8) for n in range(N))
            by = layer_bytes(N) + kv_bytes
            res[f"N{N}_T{T}"] = {"us_per_layer_tick": ms * 1e3, "launches_per_layer": 10, "tokens_per_s_through_32_layers": N / (32 * ms * 1e-3),
                                  "bytes_per_layer_tick": by, "GBps": by / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": by / (ms * 1e-3) / 1e9 / hbm_peak}
            del gr, kt, vt, kviews, vviews
        return res

    def cfg_ep():
        """C3 decode block with the experts sharded over the ranks (all-to-all dispatch and combine through the
        library's own exchange entry); 64 tokens per GPU."""
        from qb200 import ep
        return ep.bench_block(dev, g, world, rank, steps=20)

    def run_extras(names):
        out = {}
        table = {"c1": ("C1_qmv_1x4096_to_4096", cfg_c1), "sweep": ("C2_sweep", cfg_sweep), "c3": ("C3_routed_experts", cfg_c3),
                 "c4": ("C4_dense_prefill_2048x4096_to_14336", cfg_c4),
                 "c5": ("C5_decode_attention_batch16", lambda: cfg_c5(16, "16 sequences on one GPU")),
                 "tick": ("decode_layer_tick_llama3_8b", cfg_tick),
                 "a7": ("attn_times_V_transpose_false_batch16", lambda: cfg_attn_products(False)),
                 "qk": ("q_times_Kt_transpose_true_batch16", lambda: cfg_attn_products(True))}
        for nm in names:
            if nm in table and rank == 0:
                key, fn = table[nm]
                try:
                    out[key] = fn()
                except Exception as ex:  # a failing extra must not take the headline line with it
                    out[key] = {"error": f"{type(ex).__name__}: {ex}"[:300]}
                torch.cuda.empty_cache()
        if world > 1:
            dist.barrier()
            if "c5" in names and 16 % world == 0:
                try:
                    r = cfg_c5(16 // world, f"batch of 16 sharded over {world} GPUs, {16 // world} per GPU, no collective")
                except Exception as ex:
                    r = {"error": f"{type(ex).__name__}: {ex}"[:300]}
                if rank == 0:
                    out["C5_decode_attention_batch16_sharded"] = r
            if "ep" in names:
                try:
                    r = cfg_ep()
                except Exception as ex:
                    r = {"error": f"{type(ex).__name__}: {ex}"[:300]}
                if rank == 0:
                    out["C3_expert_parallel"] = r
        return out

    if only:
        res = run_extras(only)
        if rank == 0:
            print(json.dumps(res))
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    # ------------------------------------------------------------------ headline: C2 at M rows per GPU
    gr, xin, yout = build_graph(M)
    warm = max(args.warmup, 3)
    sampler = ClockSampler(local)
    for _ in range(warm * R):
        gr.replay()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps * R):
        gr.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ms = float(t.item())
    ms_step = ms / args.steps
    value = world * M * L * R * args.steps / (ms * 1e-3)

    # end to end: host buffers in, host buffers out, copies inside the timed region.  Every pass copies its inputs
    # from pinned host memory and its outputs back; two sets of device buffers (two graphs over the same weights)
    # alternate, so that the copies of one pass overlap the kernels of its neighbours, as a serving loop would run it.
    gr2, xin2, yout2 = build_graph(M)
    sets = [(gr, xin, yout), (gr2, xin2, yout2)]
    xin_h = [torch.empty(xin.shape, dtype=xin.dtype, pin_memory=True).copy_(xin) for _ in range(2)]
    yout_h = [torch.empty(yout.shape, dtype=yout.dtype, pin_memory=True) for _ in range(2)]
    s_main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    evs = [[torch.cuda.Event() for _ in range(3)] for _ in range(2)]

    def e2e_passes(n):
        used = [False, False]
        for i in range(n):
            b = i & 1
            g_b, x_b, y_b = sets[b]
            ev_in, ev_comp, ev_out = evs[b]
            with torch.cuda.stream(s_in):
                if used[b]:
                    s_in.wait_event(ev_comp)           # the kernels that read this input buffer two passes ago
                x_b.copy_(xin_h[b], non_blocking=True)
                ev_in.record(s_in)
            s_main.wait_event(ev_in)
            if used[b]:
                s_main.wait_event(ev_out)              # the read-back of this output buffer two passes ago
            g_b.replay()
            ev_comp.record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_comp)
                yout_h[b].copy_(y_b, non_blocking=True)
                ev_out.record(s_out)
            used[b] = True
        s_main.wait_stream(s_in)
        s_main.wait_stream(s_out)

    s_in.wait_stream(s_main)
    s_out.wait_stream(s_main)
    e2e_passes(8)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    e2e_passes(args.steps * R)
    e1.record()
    torch.cuda.synchronize()
    ms_e2e = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms_e2e], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item())
    clocks = sampler.stop() if rank == 0 else None
    e2e_value = world * M * L * R * args.steps / (ms_e2e * 1e-3)
    del gr2, xin2, yout2, sets

    extras = {} if args.no_configs else run_extras(["c1", "sweep", "tick", "c3", "c4", "c5", "a7", "qk"] + (["ep"] if world > 1 else []))

    if rank == 0:
        achieved = L * R * layer_bytes(M) / (ms_step * 1e-3) / 1e9
        nl = launches_per_layer(M)
        per_launch = layer_bytes(M) / (7.0 if args.no_batch else 4.0)
        out = {
            "metric": METRIC, "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": dict(CONFIG, M_per_gpu=M),
            "step": {"passes_per_step": R, "layers_per_pass": L, "weights_bytes_per_pass": L * layer_bytes(0),
                     "timed_region_s": ms * 1e-3, "parallelism": "batch-sharded x%d, weights replicated, no collective" % world,
                     "tokens_per_s_through_32_layers": value / 32.0},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "peak_source": peak_src, "frac_of_nominal_8TBs": achieved / 8000.0,
                         "bytes_per_launch": per_launch, "kernel": "qmv_stream_kernel",
                         "traffic": NCU_TRAFFIC_OVER_ALGORITHMIC * per_launch,
                         "traffic_source": "ncu dram__bytes_read+write of the four launches of one layer (2-layer "
                                           "capture), scaled by algorithmic bytes to the average launch"},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": xin.numel() * 2 * R,
                    "d2h_bytes_per_step": yout.numel() * 2 * R, "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": args.steps * R * L * nl,
            "clocks": clocks,
        }
        if clocks and clocks.get("sm_mhz"):
            out["step"]["ms_per_step_x_median_sm_mhz"] = ms_step * clocks["sm_mhz"]
        sw = extras.get("C2_sweep", {})
        if isinstance(sw, dict) and "M1" in sw:
            out["qmv_m1"] = {"us_per_layer": sw["M1"]["us_per_layer"], "tokens_per_s": sw["M1"]["tokens_per_s"],
                             "hbm_gbs": sw["M1"]["GBps"], "frac_of_peak": sw["M1"]["frac_of_hbm_peak"]}
        if extras:
            out["configs"] = extras
        if not args.no_cpu_baseline:
            cpu = CpuLayer(M)
            cpu.one_pass()
            dt1 = cpu.time_passes(1)
            n = max(1, min(50, int(12.0 / max(dt1, 1e-6))))
            dt = cpu.time_passes(n)
            out["cpu_baseline"] = {"value": M / dt, "unit": "tokens/s", "cores": cpu.qo.num_threads(), "kind": "port",
                                   "sample": f"{n} passes of one layer (7 projections) at M={M}, weights of random codes"}
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
