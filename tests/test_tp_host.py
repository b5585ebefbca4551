"""World-size-2 test of the tensor-parallel partitioning logic on CPU: two gloo ranks each compute
their row slice of the MLP block with the CPU oracle and all-gather; the result must be bit-identical
to the unsplit product (rows are independent)."""
import importlib
import os
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent

WORKER = r'''
import os, sys, importlib
import numpy as np
sys.path.insert(0, os.environ["LSPK_ROOT"])
import torch
import torch.distributed as dist
import __graft_entry__ as entry
entry.load_package()
orc = entry.load_oracle()
tp = importlib.import_module("litespark_inference_b200.torchless.tp")
synthetic = importlib.import_module("litespark_inference_b200.torchless.synthetic")

dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{os.environ['LSPK_PORT']}",
                        rank=int(os.environ["RANK"]), world_size=int(os.environ["WORLD_SIZE"]))
rank, world = dist.get_rank(), dist.get_world_size()
kern = orc.Kernels("port")
cfg = synthetic.toy_config(hidden=256, inter=512)
model = synthetic.random_model(cfg, seed=3, norm_jitter=0.1)      # same seed on every rank: replicated weights
L = model.layers[0]
x = np.random.default_rng(9).standard_normal(cfg.hidden_size).astype(np.float32)
eps = cfg.rms_norm_eps

def all_gather(v):
    parts = [torch.empty(v.shape[0], dtype=torch.float32) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(v)))
    return torch.cat(parts).numpy()

g_r, u_r, d_r = (tp.slice_projection(p, world, rank) for p in (L.gate_proj, L.up_proj, L.down_proj))

def gate_up_slice(xv):
    q8 = np.empty(xv.shape[0], np.int8)
    s = kern.rmsnorm_quantize_into(xv, L.post_attn_norm, q8, np.empty_like(xv), eps)
    g = kern.matmul_packed_m1(q8, g_r.w_packed, np.float32(g_r.scale), s)
    u = kern.matmul_packed_m1(q8, u_r.w_packed, np.float32(u_r.scale), s)
    return kern.relu2_mul_into(g, u, np.empty_like(g))

def down_slice(inter):
    q8 = np.empty(inter.shape[0], np.int8)
    s = kern.rmsnorm_quantize_into(np.ascontiguousarray(inter), L.ffn_sub_norm, q8, np.empty_like(inter), eps)
    return kern.matmul_packed_m1(q8, d_r.w_packed, np.float32(d_r.scale), s)

y = tp.mlp_block(x, L, eps, world, rank, gate_up_slice, down_slice, all_gather)

# unsplit reference on every rank
q8 = np.empty(cfg.hidden_size, np.int8)
s = kern.rmsnorm_quantize_into(x, L.post_attn_norm, q8, np.empty_like(x), eps)
g = kern.matmul_packed_m1(q8, L.gate_proj.w_packed, np.float32(L.gate_proj.scale), s)
u = kern.matmul_packed_m1(q8, L.up_proj.w_packed, np.float32(L.up_proj.scale), s)
inter = kern.relu2_mul_into(g, u, np.empty_like(g))
q2 = np.empty(inter.shape[0], np.int8)
s2 = kern.rmsnorm_quantize_into(inter, L.ffn_sub_norm, q2, np.empty_like(inter), eps)
want = kern.matmul_packed_m1(q2, L.down_proj.w_packed, np.float32(L.down_proj.scale), s2)
assert np.array_equal(y, want), "gathered TP result differs from the unsplit product"
lo, hi = tp.row_range(cfg.intermediate_size, world, rank)
assert (hi - lo) * world == cfg.intermediate_size
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_row_split_mlp_block_world2_gloo(tmp_path):
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER)
    port = _free_port()
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LSPK_PORT=str(port), LSPK_ROOT=str(ROOT),
                   OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{o}"
        assert f"rank {r} ok" in o


def test_row_range_and_slicing():
    tp = importlib.import_module("litespark_inference_b200.torchless.tp")
    synthetic = importlib.import_module("litespark_inference_b200.torchless.synthetic")
    rng = np.random.default_rng(0)
    p = synthetic.random_projection(rng, 48, 64)
    parts = [tp.slice_projection(p, 4, r) for r in range(4)]
    assert np.array_equal(np.concatenate([q.w_packed for q in parts]), p.w_packed)
    assert [tp.row_range(6912, 8, r) for r in (0, 7)] == [(0, 864), (6048, 6912)]
    import pytest
    with pytest.raises(ValueError):
        tp.row_range(10, 4, 0)
