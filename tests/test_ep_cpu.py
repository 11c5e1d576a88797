"""CPU test of the expert-parallel exchange (tie_b200/ep.py) on two gloo ranks.

The device ops are replaced by stand-ins built on the CPU restatement (oracle/), so what is
tested is the bookkeeping: counts exchange, all-to-all splits, order of rows on the way back,
combine through the dispatch permutation.  The result must equal the single-process oracle."""
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))

WORKER = r"""
import os, sys
sys.path.insert(0, %(root)r)
import numpy as np, torch, torch.distributed as dist
from tie_b200 import synth, workloads, ep
from oracle import port

rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%(port)d", rank=rank, world_size=world)
shape = synth.MoeShape(hidden=512, n_expert=32, top_k=4, ffn_dim=256)
layer = synth.make_layer(workloads.BASE_SEED + 1, shape)
P = port.PortMoe(layer)
n_local = shape.n_expert // world

class Ops:
    K, H, E = shape.top_k, shape.hidden, shape.n_expert
    def empty(self, shp, dtype): return torch.zeros(shp, dtype=dtype)
    def route(self, x, idx, w):
        i, ww, _ = P.route(x.numpy()); idx.copy_(torch.from_numpy(i)); w.copy_(torch.from_numpy(ww))
    def dispatch(self, x, idx, send_rows, send_expert, counts):
        flat = idx.numpy().reshape(-1)
        perm = np.argsort(flat, kind="stable")
        self.inv = np.empty_like(perm); self.inv[perm] = np.arange(perm.size)
        send_rows.copy_(torch.from_numpy(x.numpy()[perm // self.K]))
        send_expert.copy_(torch.from_numpy(flat[perm].astype(np.int32)))
        counts.copy_(torch.from_numpy(np.bincount(flat, minlength=self.E).astype(np.int32)))
    def expert_rows(self, rows, experts, n, y):
        if n:
            e = experts.numpy()[:n]
            assert ((e >= rank * n_local) & (e < (rank + 1) * n_local)).all(), "row sent to the wrong rank"
            y[:n].copy_(torch.from_numpy(P.expert_rows(rows.numpy()[:n], e)))
    def combine(self, y_sorted, w, out):
        ys = y_sorted.numpy()[self.inv].reshape(w.shape[0], self.K, self.H)
        acc = np.zeros((w.shape[0], self.H), dtype=np.float32)
        for j in range(self.K):
            acc = (w.numpy()[:, j:j+1].astype(np.float64) * ys[:, j].astype(np.float64) + acc.astype(np.float64)).astype(np.float32)
        out.copy_(torch.from_numpy(acc))

T = %(tokens)d
x = synth.make_x(workloads.BASE_SEED + 1, T, shape.hidden, first_token=rank * T)
blk = ep.EpMoeBlock(Ops(), torch, dist)
out = blk.forward(torch.from_numpy(x)).numpy()
ref, _, _ = P.moe_ffn(x)
err = float(workloads.rel_rms_err(out, ref).max())
assert err < 1e-6, err
assert sum(blk.last["send_counts"]) == T * shape.top_k
tot = torch.tensor([blk.last["rows_received"]]); dist.all_reduce(tot)
assert int(tot.item()) == world * T * shape.top_k
dist.barrier(); dist.destroy_process_group()
print("EP_OK", rank, err)
"""


@pytest.mark.parametrize("tokens", [1, 13])
def test_exchange_matches_single_process_oracle(tokens, tmp_path):
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    code = WORKER % dict(root=ROOT, port=port, tokens=tokens)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "EP_OK" in o, f"rank {r}:\n{o[-3000:]}"


# The peer-memory path (csrc/ep.cu) has no collective: every rank derives the whole row layout
# from the G x E count matrix.  Here two gloo ranks run ep.peer_layout (the host restatement of
# that index arithmetic) with "peer memory" stood in by all_gather'ed arrays, and the combined
# result must equal the single-process oracle: an error in the segment / output-position algebra
# sends some row to the wrong expert or token.
PEER_WORKER = r"""
import os, sys
sys.path.insert(0, %(root)r)
import numpy as np, torch, torch.distributed as dist
from tie_b200 import synth, workloads, ep
from oracle import port

rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%(port)d", rank=rank, world_size=world)
shape = synth.MoeShape(hidden=512, n_expert=32, top_k=4, ffn_dim=256)
layer = synth.make_layer(workloads.BASE_SEED + 1, shape)
P = port.PortMoe(layer)
K, H, E = shape.top_k, shape.hidden, shape.n_expert
NL = E // world
T = %(tokens)d + 3 * rank          # ragged: the ranks bring different token counts
x = synth.make_x(workloads.BASE_SEED + 1, T, H, first_token=100 * rank)

# publish: route, stable sort of the (token, slot) rows by expert, counts
idx, w, _ = P.route(x)
flat = idx.reshape(-1)
ids = np.argsort(flat, kind="stable").astype(np.int32)
counts = np.bincount(flat, minlength=E).astype(np.int32)

def gather(obj):
    out = [None] * world
    dist.all_gather_object(out, obj)
    return out

peer_counts, peer_ids, peer_x = gather(counts), gather(ids), gather(x)   # what the owners read from the sources
L = ep.peer_layout(np.stack(peer_counts), rank)

# compute: rows of this rank's experts, gathered per segment from their sources; every row
# remembers (source rank, row id there): that is where its output is stored
n = L["n_rows"]
rows = np.zeros((n, H), dtype=np.float32); experts = np.zeros(n, dtype=np.int32)
dst = np.zeros((n, 2), dtype=np.int64)
for i in range(NL * world):
    le, s = divmod(i, world)
    b, e = int(L["seg_base"][i]), int(L["seg_base"][i + 1])
    assert e - b == peer_counts[s][rank * NL + le]
    for j in range(e - b):
        rid = peer_ids[s][int(L["seg_src"][i]) + j]
        rows[b + j] = peer_x[s][rid // K]
        experts[b + j] = rank * NL + le
        dst[b + j] = (s, rid)
y = P.expert_rows(rows, experts) if n else np.zeros((0, H), dtype=np.float32)
delivered = gather((dst, y))                                             # the owners' stores into the sources' y

# gather: out[t] = sum_j w[t][j] * y[t*K + j], j ascending, on the rows the owners delivered
y_mine = np.full((T * K, H), np.nan, dtype=np.float32)
for d_dst, d_y in delivered:
    for (s, rid), row in zip(d_dst, d_y):
        if s == rank:
            assert np.isnan(y_mine[rid]).all(), "row delivered twice"
            y_mine[rid] = row
assert not np.isnan(y_mine).any(), "row never delivered"
acc = np.zeros((T, H), dtype=np.float32)
for t in range(T):
    for j in range(K):
        acc[t] = (np.float64(w[t, j]) * y_mine[t * K + j].astype(np.float64) + acc[t].astype(np.float64)).astype(np.float32)
ref, _, _ = P.moe_ffn(x)
err = float(workloads.rel_rms_err(acc, ref).max()) if T else 0.0
assert err < 1e-6, err
tot = torch.tensor([n]); dist.all_reduce(tot)
assert int(tot.item()) == sum(int(c.sum()) for c in peer_counts)
dist.barrier(); dist.destroy_process_group()
print("EP_OK", rank, err)
"""


@pytest.mark.parametrize("tokens", [0, 11])
def test_peer_layout_matches_single_process_oracle(tokens):
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    code = PEER_WORKER % dict(root=ROOT, port=port, tokens=tokens)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "EP_OK" in o, f"rank {r}:\n{o[-3000:]}"


# Decode under expert parallelism keeps the tokens replicated: every rank routes the same token,
# computes the down rows of the slots whose experts it owns and hands them to every rank; each rank
# then combines ALL slots in slot order.  Two gloo ranks do that with the CPU restatement standing
# in for the kernels and all_gather for the peer stores: every slot must be delivered exactly once,
# and the result must be the single-process oracle's, bit for bit (same order of additions).
DECODE_WORKER = r"""
import os, sys
sys.path.insert(0, %(root)r)
import numpy as np, torch, torch.distributed as dist
from tie_b200 import synth, workloads
from oracle import port

rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%(port)d", rank=rank, world_size=world)
shape = synth.MoeShape(hidden=512, n_expert=32, top_k=4, ffn_dim=256)
layer = synth.make_layer(workloads.BASE_SEED + 1, shape)
P = port.PortMoe(layer)
K, H, E = shape.top_k, shape.hidden, shape.n_expert
NL = E // world
T = %(tokens)d
x = synth.make_x(workloads.BASE_SEED + 1, T, H, first_token=40)       # the SAME tokens on every rank
idx, w, _ = P.route(x)                                                 # redundant routing
flat = idx.reshape(-1)
mine = np.nonzero((flat >= rank * NL) & (flat < (rank + 1) * NL))[0]   # (token, slot) rows this rank owns
y_loc = P.expert_rows(x[mine // K], flat[mine]) if mine.size else np.zeros((0, H), dtype=np.float32)
parts = [None] * world
dist.all_gather_object(parts, (mine, y_loc))                           # the stores into every rank's y rows
y = np.full((T * K, H), np.nan, dtype=np.float32)
for rows, vals in parts:
    for r, v in zip(rows, vals):
        assert np.isnan(y[r]).all(), "slot delivered twice"
        y[r] = v
assert not np.isnan(y).any(), "slot never delivered"
acc = np.zeros((T, H), dtype=np.float32)
for t in range(T):
    for j in range(K):
        acc[t] = (np.float64(w[t, j]) * y[t * K + j].astype(np.float64) + acc[t].astype(np.float64)).astype(np.float32)
ref, ref_idx, _ = P.moe_ffn(x)
assert np.array_equal(idx, ref_idx)
err = float(workloads.rel_rms_err(acc, ref).max())
assert err < 1e-6, err
dist.barrier(); dist.destroy_process_group()
print("EP_OK", rank, err)
"""


@pytest.mark.parametrize("tokens", [1, 4])
def test_replicated_decode_matches_single_process_oracle(tokens):
    import socket
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    code = DECODE_WORKER % dict(root=ROOT, port=port, tokens=tokens)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "EP_OK" in o, f"rank {r}:\n{o[-3000:]}"
