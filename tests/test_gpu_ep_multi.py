"""Expert parallelism over peer memory on real peers: one process per GPU (needs >= 2 GPUs; the
single-GPU emulation of the same protocol is tests/test_gpu_ep_peer.py).  The handles of the
regions travel over gloo; no collective library touches the data path."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))

WORKER = r"""
import os, sys
sys.path.insert(0, %(root)r)
import numpy as np, torch, torch.distributed as dist
from tie_b200 import synth, workloads, ep, moe
from oracle import port

rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%(port)d", rank=rank, world_size=world)
shape = synth.MoeShape()
n_local = shape.n_expert // world
silu = np.fromfile(os.path.join(%(root)r, "tests", "golden", "silu_table_ref.f32"), dtype=np.float32)
T_MAX = 128
be = moe.MoeBackend(max_tokens=T_MAX * world, device=rank, silu_table=silu, ep_rank=rank, ep_size=world)
be.upload_layer(0, synth.make_layer(workloads.BASE_SEED, shape, first_expert=rank * n_local, n_local_expert=n_local))
stream = torch.cuda.Stream(); torch.cuda.set_stream(stream); be.set_stream(stream.cuda_stream)
blk = ep.PeerEpMoeBlock(be, dist)
P = port.PortMoe(synth.make_layer(workloads.BASE_SEED, shape), silu=silu)
worst = 0.0
for step, T in enumerate([96, 128, 1 + 40 * rank, 64]):       # ragged third step
    x = synth.make_x(workloads.BASE_SEED + step, T, shape.hidden, first_token=500 * rank)
    xd = torch.from_numpy(x).cuda(); od = torch.full_like(xd, float("nan"))
    stream.synchronize()
    dist.barrier()                                             # hosts start a step together; the devices then free-run
    blk.forward(xd, od)
    be.synchronize()                                           # also reads the device status word
    ref, _, _ = P.moe_ffn(x)
    err = float(workloads.rel_rms_err(od.cpu().numpy(), ref).max())
    assert err < 1e-3, (step, err)
    worst = max(worst, err)
# two chained blocks in place (RMSNorm, experts over both GPUs, residual), each step one graph replay
h_host = synth.make_x(workloads.BASE_SEED + 9, 64, shape.hidden, first_token=300 * rank)
hd = torch.from_numpy(h_host).cuda()
for rep in range(2):
    stream.synchronize(); dist.barrier()
    be.moe_block_inplace_ep_ptr(0, hd, 64, moe.DEVICE | moe.NO_SYNC | moe.GRAPH)
be.synchronize()
R = port.PortMoe(synth.make_layer(workloads.BASE_SEED, shape), silu=silu)
want = h_host.copy()
for rep in range(2):
    want = R.moe_block_inplace(want)[0]
err = float(workloads.rel_rms_err(hd.cpu().numpy(), want).max())
assert err < 1e-3, ("block_inplace_ep", err)
dist.barrier()
be.close()
dist.destroy_process_group()
print("EP_OK", rank, worst)
"""


def test_two_gpus_match_the_oracle():
    import socket
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    code = WORKER % dict(root=ROOT, port=port)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", OMP_NUM_THREADS="4")
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=600)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "EP_OK" in o, f"rank {r}:\n{o[-3000:]}"
