"""Expert parallelism for the MoE block: one process per GPU, experts sharded 128/G per rank,
tokens data-parallel.  The reference is a single process and has no counterpart.

Two exchanges are implemented:

PeerEpMoeBlock (default)  dispatch and combine over peer memory (tie_cuda_ep_*): every rank exposes
    one region of its HBM; a rank stores its tokens into every rank's region while it routes them,
    and the down product stores every output row straight into its source's region (plain stores
    over NVLink; only the small row lists are loaded), synchronised by step-numbered flags.  No collective and no host
    synchronisation per step; torch.distributed only exchanges the IPC handles once.

EpMoeBlock (baseline)     the same step with NCCL collectives (torch.distributed):
      route (local, router replicated)                       -> top-k ids, weights
      dispatch: counting sort of the (token, slot) rows by expert id; since a rank owns a
                contiguous expert range this also groups rows by destination rank
      all-to-all of the per-expert row counts (to each expert's owner), then of the rows
      expert rows on the owner (grouped mat-vec / GEMM over its local experts)
      all-to-all back in the same order
      combine: out[t] = sum_j w[t][j] * y[(t, j)], j ascending
    Its exchange logic is written against a small `ops` interface so that it can run on CPU ranks
    (gloo) with stand-in ops in the tests; on GPUs `CudaOps` forwards to the C ABI.
"""
from __future__ import annotations

import json
import os

import numpy as np


class CudaOps:
    """Device ops of one rank, forwarding to libtie_cuda.so."""

    def __init__(self, be, torch):
        self.be, self.torch = be, torch
        self.K, self.H, self.E = be.top_k, be.hidden, be.n_expert
        self.device = torch.device("cuda", be.cfg.device)

    def empty(self, shape, dtype):
        return self.torch.empty(shape, dtype=dtype, device=self.device)

    def route(self, x, idx, w):
        from . import moe
        self.be.route_ptr(0, x, x.shape[0], idx, w, None, None, moe.DEVICE | moe.NO_SYNC)

    def dispatch(self, x, idx, send_rows, send_expert, counts):
        from . import moe
        self.be.ep_dispatch_ptr(x, idx, x.shape[0], send_rows, send_expert, counts, moe.DEVICE | moe.NO_SYNC)

    def expert_rows(self, rows, experts, n_rows, y):
        from . import moe
        if n_rows:
            self.be.expert_rows_ptr(0, rows, experts, n_rows, y, moe.DEVICE | moe.NO_SYNC)

    def combine(self, y_sorted, w, out):
        from . import moe
        self.be.ep_combine_ptr(y_sorted, w, out.shape[0], out, moe.DEVICE | moe.NO_SYNC)


class EpMoeBlock:
    """One expert-parallel MoE block on this rank.  ops supplies route / dispatch / expert_rows /
    combine; dist is torch.distributed (any backend with all_to_all_single)."""

    def __init__(self, ops, torch, dist, group=None):
        self.ops, self.torch, self.dist, self.group = ops, torch, dist, group
        self.G = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.n_local = ops.E // self.G
        self.last = {}

    def forward(self, x, out=None):
        torch, dist, ops = self.torch, self.dist, self.ops
        T, K, H, G = x.shape[0], ops.K, ops.H, self.G
        R = T * K
        idx = ops.empty((T, K), torch.int32)
        w = ops.empty((T, K), torch.float32)
        ops.route(x, idx, w)
        send_rows = ops.empty((R, H), torch.float32)
        send_expert = ops.empty((R,), torch.int32)
        counts = ops.empty((ops.E,), torch.int32)
        ops.dispatch(x, idx, send_rows, send_expert, counts)
        # per-expert row counts go to the expert's owner: every rank then knows how many rows it
        # receives from whom AND, the rows of a source being sorted by expert, which expert each
        # received row belongs to (no second exchange for the ids)
        recv_mat = torch.empty_like(counts)  # [source rank][local expert]
        dist.all_to_all_single(recv_mat, counts, group=self.group)
        send_counts = counts.view(G, self.n_local).sum(dim=1)
        recv_counts = recv_mat.view(G, self.n_local).sum(dim=1)
        both = torch.cat([send_counts, recv_counts]).tolist()  # host sync: split sizes are host arguments of the collective
        sc, rc = both[:G], both[G:]
        n_recv = int(sum(rc))
        recv_rows = ops.empty((max(n_recv, 1), H), torch.float32)
        dist.all_to_all_single(recv_rows[:n_recv], send_rows, rc, sc, group=self.group)
        local_ids = torch.arange(self.rank * self.n_local, (self.rank + 1) * self.n_local, dtype=torch.int32, device=counts.device)
        recv_expert = ops.empty((max(n_recv, 1),), torch.int32)
        if n_recv:
            recv_expert[:n_recv] = torch.repeat_interleave(local_ids.repeat(G), recv_mat.to(torch.int64), output_size=n_recv)
        y_recv = ops.empty((max(n_recv, 1), H), torch.float32)
        ops.expert_rows(recv_rows, recv_expert, n_recv, y_recv)
        y_sorted = ops.empty((R, H), torch.float32)
        dist.all_to_all_single(y_sorted, y_recv[:n_recv], sc, rc, group=self.group)
        if out is None:
            out = ops.empty((T, H), torch.float32)
        ops.combine(y_sorted, w, out)
        self.last = {"rows_sent": R, "rows_received": n_recv, "send_counts": sc, "recv_counts": rc}
        return out


def peer_layout(counts, rank: int, n_tile: int = 64):
    """Host restatement of the row layout the peer-memory path derives on the device (ep_index in
    csrc/ep.cu) from the G x E matrix counts[s][e] = rows of source rank s for global expert e.

    Returns a dict with, for `rank` (owner of experts [rank*NL, (rank+1)*NL)):
      offsets[NL+1]   first sorted row of each local expert (rows ordered by expert, then source)
      tiles           (local expert, first row, rows) per token tile of n_tile rows
      seg_base[NL*G+1], seg_src[NL*G]  segment le*G+s: its first row here, its first entry in s's id list
    Row j of segment (le, s) is row id ids_s[seg_src + j] of rank s: its token row is read from
    there and its output is stored there, at that row id.
    """
    counts = np.asarray(counts, dtype=np.int64)
    G, E = counts.shape
    NL = E // G
    fe = rank * NL
    tot = counts.sum(axis=0)
    offsets = np.concatenate([[0], np.cumsum(tot[fe:fe + NL])])
    tiles = [(le, int(offsets[le]) + j, int(min(n_tile, tot[fe + le] - j)))
             for le in range(NL) for j in range(0, int(tot[fe + le]), n_tile)]
    src_off = np.concatenate([np.zeros((G, 1), dtype=np.int64), np.cumsum(counts, axis=1)], axis=1)  # [G][E+1]
    seg_base = np.zeros(NL * G + 1, dtype=np.int64)
    seg_src = np.zeros(NL * G, dtype=np.int64)
    for le in range(NL):
        for s in range(G):
            seg_base[le * G + s] = offsets[le] + counts[:s, fe + le].sum()
            seg_src[le * G + s] = src_off[s, fe + le]
    seg_base[NL * G] = offsets[NL]
    return {"offsets": offsets, "tiles": tiles, "seg_base": seg_base, "seg_src": seg_src, "n_rows": int(offsets[NL])}


class PeerEpMoeBlock:
    """One expert-parallel MoE block on this rank over peer memory (tie_cuda_ep_*): no collective
    and no host synchronisation per step.  torch.distributed is used once, to exchange the IPC
    handles of the ranks' regions."""

    def __init__(self, be, dist, group=None):
        from . import moe
        self.be, self.moe = be, moe
        G = dist.get_world_size(group)
        handles = [None] * G
        dist.all_gather_object(handles, be.ep_ipc_handle(), group=group)
        be.ep_attach(handles, moe.EP_PEER_IPC_HANDLES)
        dist.barrier(group=group)  # every rank has mapped every region before the first flag is written

    def forward(self, x, out, graph: bool = True):
        """x, out: device tensors [n_tokens][hidden].  graph: replay the step's launches from a CUDA
        graph (one per distinct (x, out, n_tokens))."""
        flags = self.moe.DEVICE | self.moe.NO_SYNC | (self.moe.GRAPH if graph else 0)
        self.be.moe_ffn_ep_ptr(0, x, out, x.shape[0], flags)
        return out

    def token_buffer(self, torch, n_tokens: int):
        """A [n_tokens][hidden] fp32 tensor over the token buffer at the start of this rank's region
        (where tie_cuda_moe_block_inplace_ep writes the normed rows)."""
        base, _ = self.be.ep_region()

        class _View:
            __cuda_array_interface__ = {"shape": (n_tokens, self.be.hidden), "typestr": "<f4", "data": (base, False), "version": 2}

        return torch.as_tensor(_View(), device=torch.device("cuda", self.be.cfg.device))


NVLINK_GBS = 770.0  # measured peer-copy rate per direction on this pool's B200s


def bind_host_threads_to_gpu(torch, device_index: int):
    """Keeps this process on the CPU cores next to its GPU (the affinity NVML reports for the device),
    so that the pinned host buffers it allocates afterwards and the threads that fill them sit on the
    GPU's side of the machine.  Reads NVML only; changes nothing but this process's own affinity.
    Returns the number of cores kept, or None where NVML or the call is unavailable."""
    try:
        import pynvml
        pynvml.nvmlInit()
        props = torch.cuda.get_device_properties(device_index)
        bus_id = f"{props.pci_domain_id:08x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus_id.encode())
        allowed = os.sched_getaffinity(0)
        n_cpu = max(max(allowed) + 1, os.cpu_count() or 1)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (n_cpu + 63) // 64)
        near = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        cores = near & allowed
        if not cores:
            return None
        os.sched_setaffinity(0, cores)
        return len(cores)
    except Exception:
        return None


def _nvlink_bytes_per_direction(shape, tokens_per_rank, world):
    """What one rank sends (and, by symmetry, receives) per step: its tokens to every peer, and the
    output rows it computed for other ranks' tokens ((world-1)/world of its rows on average)."""
    row = shape.hidden * 4
    return tokens_per_rank * row * (world - 1) + tokens_per_rank * shape.top_k * row * (world - 1) / world


def _step_roofline(shape, tokens_per_rank, world, ms_per_step, flops_total, peaks):
    nvlink_bytes = _nvlink_bytes_per_direction(shape, tokens_per_rank, world)
    hbm_bytes = (shape.n_expert // world) * shape.expert_bytes + shape.router_bytes + 2 * tokens_per_rank * shape.hidden * 4
    t_nvlink = nvlink_bytes / (NVLINK_GBS * 1e9)
    t_hbm = hbm_bytes / (peaks["hbm_gbs"] * 1e9)
    t_tensor = (flops_total / world) / (peaks["bf16_tflops"] * 1e12)
    floors = {"nvlink": t_nvlink, "hbm": t_hbm, "tensor": t_tensor}
    bound = max(floors, key=floors.get)
    t = ms_per_step * 1e-3
    if bound == "nvlink":
        achieved, peak, unit = nvlink_bytes / t / 1e9, NVLINK_GBS, "GB/s"
    elif bound == "hbm":
        achieved, peak, unit = hbm_bytes / t / 1e9, peaks["hbm_gbs"], "GB/s"
    else:
        achieved, peak, unit = flops_total / world / t / 1e12, peaks["bf16_tflops"], "TFLOP/s"
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak, "traffic": None,
            "floors_us": {k: v * 1e6 for k, v in floors.items()},
            "nvlink": {"bytes_per_direction": nvlink_bytes, "achieved_gbs": nvlink_bytes / t / 1e9, "peak_gbs": NVLINK_GBS},
            "note": "one rank's whole step against the slowest of its floors (tokens and output rows over NVLink in one direction at the measured "
                    "770 GB/s peer copy, algorithmic HBM bytes at the measured copy rate, flops at the measured bf16 GEMM rate); "
                    "the per-kernel HBM roofline is reported by the 1-GPU run",
            "algorithmic_tflops": flops_total / t / 1e12}


def sample_rows(n_rows: int, n: int = 8):
    """Row indices checked after a benchmark run: first, last and evenly spaced ones between."""
    if n_rows <= n:
        return list(range(n_rows))
    return sorted({0, n_rows - 1, *[(i * (n_rows - 1)) // (n - 1) for i in range(1, n - 1)]})


PARITY_TOL = 1e-3


def bench_main(args, metric, unit, tokens_per_rank, load_peaks, ClockSampler, config_of, cpu_baseline_leg, row_checker):
    """bench.py --gpus N under torchrun: weak scaling, `tokens_per_rank` tokens on every rank,
    experts sharded.  Rank 0 prints the JSON line.  row_checker(seed, x_rows, got_rows, block) ->
    max over the rows of max_k|got - want| / rms_k(want), `want` from the caller's CPU checker
    (block: the rows are residual-stream rows of h += MoE(RMSNorm(h))); it is called outside the
    timed regions on a few rows of every rank."""
    import torch
    import torch.distributed as dist

    from . import moe, synth, workloads

    world = int(os.environ["WORLD_SIZE"])
    rank = int(os.environ["RANK"])
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local_rank)
    near_cores = bind_host_threads_to_gpu(torch, local_rank)  # before any pinned allocation
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    shape = synth.MoeShape()
    T = tokens_per_rank
    n_local = shape.n_expert // world
    layer = synth.make_layer(workloads.BASE_SEED, shape, first_expert=rank * n_local, n_local_expert=n_local)
    STRONG_TOKENS = 8192  # side run: BASELINE's expert-parallel prefill, 8192 tokens in total whatever N
    cap = max(T * world, STRONG_TOKENS)
    be = moe.MoeBackend(max_tokens=cap, device=local_rank, silu_table=moe.silu_table_default(), ep_rank=rank, ep_size=world)
    be.upload_layer(0, layer)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    be.set_stream(stream.cuda_stream)
    exchange = getattr(args, "ep_exchange", "peer")
    if exchange == "peer":
        blk = PeerEpMoeBlock(be, dist)
    else:
        nccl_blk = EpMoeBlock(CudaOps(be, torch), torch, dist)

        class _Adapter:
            last = nccl_blk.last

            def forward(self, x, out):
                return nccl_blk.forward(x, out)

        blk = _Adapter()

    x_host = torch.from_numpy(synth.make_x(workloads.BASE_SEED, T, first_token=rank * T)).pin_memory()
    out_host = torch.empty_like(x_host).pin_memory()
    if exchange == "peer":
        x_dev = blk.token_buffer(torch, T)  # (any device buffer would do: the step hands the tokens to the peers itself)
        x_dev.copy_(x_host)
    else:
        x_dev = x_host.cuda()
    out_dev = torch.empty_like(x_dev)

    def step():
        blk.forward(x_dev, out_dev)

    def step_e2e():
        x_dev.copy_(x_host, non_blocking=True)
        blk.forward(x_dev, out_dev)
        out_host.copy_(out_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    l0 = be.launch_count
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    launches = be.launch_count - l0
    clocks = sampler.stop() if rank == 0 else None
    total_ms = float(ms.item())

    def timed(fn, n):
        """ms per call of fn over n calls: CUDA events on this rank's stream, max over ranks."""
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / n

    for _ in range(args.warmup):
        step_e2e()
    e2e_sync_s = timed(step_e2e, args.steps) * 1e-3
    be.synchronize()
    e2e_s, e2e_how = e2e_sync_s, "one step at a time: copy in, step, copy out in series"
    if exchange == "peer":
        # three steps in flight on device and host buffers used in turn: every step still copies its tokens
        # in and its result out inside the timed region, and the host waits for each step's result; the
        # copies run on streams of their own and overlap the neighbouring steps' kernels
        DEPTH = 3
        cs = torch.cuda.current_stream()
        hs, ds = torch.cuda.Stream(), torch.cuda.Stream()
        xb = [torch.empty(T, shape.hidden, device="cuda") for _ in range(DEPTH)]
        ob = [torch.empty_like(b) for b in xb]
        xh = [x_host] + [x_host.clone().pin_memory() for _ in range(DEPTH - 1)]
        oh = [out_host] + [torch.empty_like(out_host).pin_memory() for _ in range(DEPTH - 1)]
        ev_in, ev_done, ev_out = ([torch.cuda.Event() for _ in range(DEPTH)] for _ in range(3))

        def pipelined(n=1):
            for i in range(n):
                k = i % DEPTH
                if i >= DEPTH:
                    ev_out[k].synchronize()  # the result of the step that used these buffers is in host memory
                with torch.cuda.stream(hs):
                    hs.wait_event(ev_done[k])
                    xb[k].copy_(xh[k], non_blocking=True)
                    ev_in[k].record(hs)
                cs.wait_event(ev_in[k])
                cs.wait_event(ev_out[k])
                blk.forward(xb[k], ob[k])
                ev_done[k].record(cs)
                with torch.cuda.stream(ds):
                    ds.wait_event(ev_done[k])
                    oh[k].copy_(ob[k], non_blocking=True)
                    ev_out[k].record(ds)
            for k in range(DEPTH):
                ev_out[k].synchronize()
                cs.wait_event(ev_out[k])

        pipelined(max(args.warmup, 4))
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        pipelined(args.steps)
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item()) / args.steps * 1e-3
        e2e_how = f"{DEPTH} steps in flight on buffers used in turn (copies on streams of their own, host waits for every step's result)"
        assert all(torch.equal(oh[0], o) for o in oh[1:]) and bool(torch.isfinite(oh[0]).all())
        be.synchronize()

    # per-phase device times of rank 0 (CUDA events inside the library; the steps run without a graph,
    # and every rank starts them together, so waits for peers show up in the phase that waits)
    phases = None
    if exchange == "peer":
        be.set_profiling(True)
        acc = None
        n_prof = 10
        for _ in range(n_prof):
            dist.barrier()
            blk.forward(x_dev, out_dev)
            prof, _ = be.get_profile()
            acc = prof if acc is None else {k: acc[k] + v for k, v in prof.items()}
        be.set_profiling(False)
        names = {"router": "router (+ tokens to the peers)", "sort": "sort + publish", "split": "wait for the peers' lists + row layout", "gate_up": "gate/up product",
                 "swiglu": "SwiGLU pass", "down": "down product (stores rows to their sources)", "combine": "wait for owners + combine"}
        phases = {names[k]: v / n_prof for k, v in acc.items()}

    # ---- parity of this rank's output rows against the CPU checker (outside every timed region) ----
    parity_rows, parity_err = 0, 0.0

    def check(seed, x_rows_host, got_dev, rows, block=False):
        nonlocal parity_rows, parity_err
        got = got_dev[rows].cpu().numpy()
        err = float(row_checker(seed, x_rows_host[rows], got, block))
        parity_rows += len(rows)
        parity_err = max(parity_err, err)
        return err

    out_dev.fill_(float("nan"))
    step()
    torch.cuda.synchronize()
    parity_detail = {"weak_step": check(workloads.BASE_SEED, x_host.numpy(), out_dev, sample_rows(T))}

    strong = None
    if exchange == "peer" and not getattr(args, "no_extra", False) and STRONG_TOKENS % world == 0:
        T2 = STRONG_TOKENS // world
        x2 = blk.token_buffer(torch, T2)
        x2_host = synth.make_x(workloads.BASE_SEED, T2, first_token=rank * T2)
        x2.copy_(torch.from_numpy(x2_host))
        o2 = torch.empty_like(x2)
        for _ in range(3):
            blk.forward(x2, o2)
        ms2 = timed(lambda: blk.forward(x2, o2), max(5, args.steps // 2))
        strong = {"tokens": STRONG_TOKENS, "tokens_per_rank": T2, "scaling": "strong", "ms_per_step": ms2,
                  "tokens_per_s": STRONG_TOKENS / (ms2 * 1e-3),
                  "algorithmic_tflops": workloads.algorithmic_flops(shape, STRONG_TOKENS) / (ms2 * 1e-3) / 1e12}
        be.synchronize()
        o2.fill_(float("nan"))
        blk.forward(x2, o2)
        torch.cuda.synchronize()
        parity_detail["strong_8192_step"] = check(workloads.BASE_SEED, x2_host, o2, sample_rows(T2))

    # side run: the 48-block stack (BASELINE's last configuration), a 4096-token prefill with the
    # tokens and the experts of every block spread over the ranks; h += MoE(RMSNorm(h)) per block
    stack = None
    n_layers = getattr(args, "stack_layers", 0)
    if exchange == "peer" and not getattr(args, "no_extra", False) and n_layers > 0 and 4096 % world == 0:
        T3 = 4096 // world
        be.synchronize()
        be2 = moe.MoeBackend(max_tokens=4096, device=local_rank, silu_table=moe.silu_table_default(), ep_rank=rank, ep_size=world,
                             n_layers=n_layers)
        ones = np.ones(shape.hidden, dtype=np.float32)
        for l in range(n_layers):
            be2.upload_layer(l, synth.make_layer(workloads.STACK_BASE_SEED + l, shape, first_expert=rank * n_local,
                                                 n_local_expert=n_local), ffn_norm_w=ones)
        be2.set_stream(stream.cuda_stream)
        PeerEpMoeBlock(be2, dist)
        h0_host = synth.make_x(workloads.STACK_BASE_SEED, T3, first_token=rank * T3)
        h0 = torch.from_numpy(h0_host).cuda()
        h = h0.clone()
        fl = moe.DEVICE | moe.NO_SYNC | moe.GRAPH

        def stack_pass():
            for l in range(n_layers):
                be2.moe_block_inplace_ep_ptr(l, h, T3, fl)

        for _ in range(2):
            h.copy_(h0)
            stack_pass()
        be2.synchronize()
        h.copy_(h0)
        ms3 = timed(stack_pass, 3)
        be2.synchronize()
        finite = bool(torch.isfinite(h).all().item())
        fl3 = workloads.algorithmic_flops(shape, 4096) * n_layers
        stack = {"layers": n_layers, "tokens": 4096, "tokens_per_rank": T3, "scaling": "strong", "ms": ms3,
                 "tokens_per_s": 4096 / (ms3 * 1e-3), "algorithmic_tflops": fl3 / (ms3 * 1e-3) / 1e12, "finite": finite,
                 "weight_bytes_per_rank": be2.weight_bytes}
        # block 0 alone on fresh rows, against the checker's h + MoE(RMSNorm(h))
        h.copy_(h0)
        be2.moe_block_inplace_ep_ptr(0, h, T3, fl)
        be2.synchronize()
        parity_detail["stack_block_0"] = check(workloads.STACK_BASE_SEED, h0_host, h, sample_rows(T3), block=True)

        # batch-1 decode through the same stack: the token is replicated, every rank routes it, runs
        # the selected experts it owns and all ranks combine the eight slots (TIE_CUDA_EP_REPLICATED)
        d0_host = synth.make_x(workloads.STACK_BASE_SEED, 1)
        d0 = torch.from_numpy(d0_host).cuda()
        d = d0.clone()
        fd = fl | moe.EP_REPLICATED
        decode_steps = 256

        def decode_pass():
            for l in range(n_layers):
                be2.moe_block_inplace_ep_ptr(l, d, 1, fd)

        for _ in range(3):
            decode_pass()
        be2.synchronize()
        d.copy_(d0)
        ms4 = timed(decode_pass, decode_steps)
        be2.synchronize()
        by = workloads.algorithmic_bytes(shape, 1, shape.top_k) * n_layers
        stack["decode"] = {"steps": decode_steps, "us_per_token": ms4 * 1e3, "tokens_per_s": 1.0 / (ms4 * 1e-3),
                           "algorithmic_bytes_per_token": by, "hbm_gbs_all_ranks": by / (ms4 * 1e-3) / 1e9,
                           "finite": bool(torch.isfinite(d).all().item()),
                           "note": "token replicated, redundant routing, each rank runs the selected experts it owns, "
                                   "down rows stored to every rank, slot-order combine on every rank"}
        d.copy_(d0)
        be2.moe_block_inplace_ep_ptr(0, d, 1, fd)
        be2.synchronize()
        parity_detail["stack_decode_block_0"] = check(workloads.STACK_BASE_SEED, d0_host, d, [0], block=True)
        dist.barrier()
        be2.close()

    pt = torch.tensor([parity_err, float(parity_rows)], device="cuda", dtype=torch.float64)
    perr = pt[:1].clone()
    prow = pt[1:].clone()
    dist.all_reduce(perr, op=dist.ReduceOp.MAX)
    dist.all_reduce(prow, op=dist.ReduceOp.SUM)
    parity = {"max_rel_rms": float(perr.item()), "rows": int(prow.item()), "tol": PARITY_TOL,
              "checker": "CPU restatement of the reference's MoE branch (bit-identical to the compiled reference), "
                         "sampled rows of every rank: first, last, evenly spaced",
              "rank0": parity_detail}
    cpu = None
    if rank == 0 and not getattr(args, "no_cpu", False):
        cpu = cpu_baseline_leg(synth.make_layer(workloads.BASE_SEED, shape), moe.silu_table_default())
    dist.barrier()

    if rank == 0:
        peaks = load_peaks()
        ms_per_step = total_ms / args.steps
        value = T * world / (ms_per_step * 1e-3)
        flops = workloads.algorithmic_flops(shape, T * world)
        line = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": config_of(shape, T * world, world),
            "config_detail": {
                "l2": f"weights touched per step per rank: {392 // world} MB plus {T * shape.top_k * shape.hidden * 8 // 2**20} MB of rows "
                      "(larger than L2 from N = 1 to 2; at N >= 4 the weights of a rank fit in L2, as they would in deployment)",
                "exchange": ("peer memory: a rank stores its tokens into every rank's HBM beside its router, owners store output rows "
                             "into the sources' (no collective, no host synchronisation per step)") if exchange == "peer"
                else "NCCL all-to-all (torch.distributed) for dispatch and combine",
                "host": f"rank 0 bound to the {near_cores} cores next to its GPU" if near_cores else "no core binding"},
            "clocks": clocks,
            "e2e": {"value": T * world / e2e_s, "unit": unit, "h2d_bytes_per_step": T * shape.hidden * 4 * world,
                    "d2h_bytes_per_step": T * shape.hidden * 4 * world, "ms_per_step": e2e_s * 1e3, "how": e2e_how,
                    "synchronous_call": {"value": T * world / e2e_sync_s, "ms_per_step": e2e_sync_s * 1e3}},
            "gpu_launches": int(launches),
            # the whole step of one rank against the slower of its three floors: rows over NVLink (one
            # direction: rows in and rows out travel opposite ways), its share of the packed weights and
            # its rows' operands from HBM, its flops on the tensor cores
            "roofline": _step_roofline(shape, T, world, ms_per_step, flops, peaks),
            "cpu_baseline": cpu,
            "parity": parity,
            "exchange": {"rows_per_rank": T * shape.top_k, "bytes_per_row": shape.hidden * 4,
                         "remote_fraction": (world - 1) / world,
                         "nvlink_bytes_per_rank_and_direction": int(_nvlink_bytes_per_direction(shape, T, world)),
                         "nvlink_floor_us": _nvlink_bytes_per_direction(shape, T, world) / (NVLINK_GBS * 1e9) * 1e6,
                         "note": "floor = tokens to every peer + output rows to their sources, of one rank / measured 770 GB/s per direction",
                         "phases_ms_rank0": phases},
            "extra": {"prefill_8192_tokens_total": strong, "stack_prefill_4096_tokens": stack},
        }
        print(json.dumps(line), flush=True)
    be.close()
    dist.destroy_process_group()
    if not (parity["max_rel_rms"] <= PARITY_TOL):
        raise SystemExit(f"expert-parallel outputs differ from the CPU checker: {parity}")
