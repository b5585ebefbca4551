"""Tensor-parallel MLP block.  On two GPUs (two child processes that meet through files): the row slices gathered
by NCCL, and then by plain stores into CUDA-IPC peer windows, must give on every rank exactly the unsplit
product.  On one GPU: the bounded wait of the peer exchange, made to run out (a one-rank group told to expect
a second rank that does not exist), reports an error code and leaves the library usable; nothing hangs."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

WORKER = r'''
import os, sys, time, importlib
import numpy as np
sys.path.insert(0, os.environ["LSPK_ROOT"])
import __graft_entry__ as entry
entry.load_package()
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
os.environ["LITESPARK_DEVICE"] = str(rank)
K = importlib.import_module("litespark_inference_b200.torchless.kernel")
dev = importlib.import_module("litespark_inference_b200.torchless.device")
tp = importlib.import_module("litespark_inference_b200.torchless.tp")
synthetic = importlib.import_module("litespark_inference_b200.torchless.synthetic")
idfile = os.environ["LSPK_IDFILE"]
if rank == 0:
    uid = tp.DeviceTP.make_unique_id()
    with open(idfile + ".tmp", "wb") as f:
        f.write(uid)
    os.replace(idfile + ".tmp", idfile)
else:
    for _ in range(600):
        if os.path.exists(idfile):
            break
        time.sleep(0.1)
    uid = open(idfile, "rb").read()
group = tp.DeviceTP(rank, world, uid)
cfg = synthetic.bitnet_2b_config(num_layers=1, vocab_size=256)
rng = np.random.default_rng(4)                                    # same stream on both ranks
gate, up = synthetic.random_projection_fast(rng, 6912, 2560), synthetic.random_projection_fast(rng, 6912, 2560)
down = synthetic.random_projection_fast(rng, 2560, 6912)
norm = synthetic.fp32_to_bf16_u16(rng.uniform(0.5, 1.5, 2560).astype(np.float32))
sub = synthetic.fp32_to_bf16_u16(rng.uniform(0.5, 1.5, 6912).astype(np.float32))
x = rng.standard_normal((1, 2560)).astype(np.float32)
W = lambda p: dev.DeviceWeight(p.w_packed, p.scale)
g_r, u_r, d_r = (W(tp.slice_projection(p, world, rank)) for p in (gate, up, down))
dx, dn, ds = dev.DeviceArray.from_numpy(x), dev.DeviceArray.from_numpy(norm), dev.DeviceArray.from_numpy(sub)
i_s, i_f = dev.DeviceArray((6912 // world,), np.float32), dev.DeviceArray((1, 6912), np.float32)
d_s, y_f = dev.DeviceArray((2560 // world,), np.float32), dev.DeviceArray((1, 2560), np.float32)
for _ in range(3):
    group.mlp_block(g_r, u_r, d_r, dx, dn, ds, 1e-5, i_s, i_f, d_s, y_f)
got = y_f.numpy()
# unsplit on this GPU
inter = dev.DeviceArray((1, 6912), np.float32)
dev.linear([W(gate), W(up)], [inter, None], 1, x_f32=dx, gamma=dn, epilogue=K.EPI_RELU2_MUL)
want = dev.DeviceArray((1, 2560), np.float32)
dev.linear([W(down)], [want], 1, x_f32=inter, gamma=ds)
assert np.array_equal(i_f.numpy(), inter.numpy()), "gathered gate/up slice differs"
assert np.array_equal(got, want.numpy()), "gathered down slice differs"

# the same block with both gathers through peer windows (CUDA IPC, plain stores, bounded waits): handles travel by file
handle = group.create_window(6912, 2560)
hfile = idfile + ".win%d" % rank
with open(hfile + ".tmp", "wb") as f:
    f.write(handle)
os.replace(hfile + ".tmp", hfile)
handles = []
for r in range(world):
    other = idfile + ".win%d" % r
    for _ in range(600):
        if os.path.exists(other):
            break
        time.sleep(0.05)
    handles.append(open(other, "rb").read())
group.open_windows(handles)
for _ in range(3):          # several exchanges: the counters only grow, epochs must keep matching
    got_peer = group.mlp_block_peer(g_r, u_r, d_r, dx, dn, ds, 1e-5, i_s, d_s)
    assert np.array_equal(got_peer, want.numpy().reshape(-1)), "peer-window result differs from the unsplit block"
    assert np.array_equal(group.window_vector(0), inter.numpy().reshape(-1)), "gathered gate product differs"
assert K.load_library(True).lspk_tc_check_error() == 0
group.close()
print("rank", rank, "ok")
'''


def _gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for ln in out.splitlines() if ln.startswith("GPU "))
    except (OSError, subprocess.TimeoutExpired):
        return 0


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_tp_mlp_block_two_gpus(tmp_path):
    script = tmp_path / "tp_gpu_worker.py"
    script.write_text(WORKER)
    idfile = tmp_path / "nccl_id.bin"
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LSPK_ROOT=str(ROOT), LSPK_IDFILE=str(idfile),
                   NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    try:
        for p in procs:
            outs.append(p.communicate(timeout=300)[0])
    finally:
        # a rank that died before the communicator was formed leaves its peer blocked inside NCCL's
        # bootstrap: never leave a child behind holding a GPU
        for p in procs:
            if p.poll() is None:
                p.kill()
                p.wait()
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, f"rank {r} failed:\n{o[-3000:]}"
        assert f"rank {r} ok" in o


def test_peer_wait_runs_out_and_reports():
    """The failure path of the peer exchange without a failing GPU: the store side of one exchange is dropped (a
    test hook), so the wait polls packets that nothing renews.  It gives up after its poll limit, the library's
    wait flag turns into LSPK_ERR_DEVICE_WAIT exactly once, the stream keeps working, and the next exchange on
    the same window succeeds.  A group whose peer window was never mapped is refused before anything launches."""
    import ctypes
    import importlib
    import numpy as np
    K = importlib.import_module("litespark_inference_b200.torchless.kernel")
    dev = importlib.import_module("litespark_inference_b200.torchless.device")
    tp = importlib.import_module("litespark_inference_b200.torchless.tp")
    lib = tp._lib()
    assert lib.lspk_tc_check_error() == 0
    buf = ctypes.create_string_buffer(64)
    sl = dev.DeviceArray.from_numpy(np.arange(32, dtype=np.float32))
    # a group of two whose second window was never mapped: the exchange refuses before launching anything
    K.check(lib.lspk_tp_window_create(0, 2, 64, 32, buf))
    lib.lspk_clear_error()
    assert lib.lspk_tp_exchange(sl.ptr, 0) == 1 and b"has not been opened" in lib.lspk_last_error()
    lib.lspk_clear_error()
    K.check(lib.lspk_tp_window_close())
    # a slice that never arrives: the test hook drops the store side of the next exchange, so its wait polls
    # packets that still carry an old exchange number
    K.check(lib.lspk_tp_window_create(0, 1, 64, 32, buf))
    K.check(lib.lspk_tp_window_set_poll_limit(2000))
    K.check(lib.lspk_tp_debug_drop_next_arrival())
    K.check(lib.lspk_tp_exchange(sl.ptr, 1))
    assert lib.lspk_tc_check_error() == 6                               # LSPK_ERR_DEVICE_WAIT, reported once
    lib.lspk_clear_error()
    assert lib.lspk_tc_check_error() == 0
    # the exchange after the lost one carries the next number: the same window works again
    full = dev.DeviceArray.from_numpy(np.arange(64, dtype=np.float32) * 0.5)
    K.check(lib.lspk_tp_exchange(sl.ptr, 1))                       # kind 1 again: the number after the lost one
    got1 = np.empty(32, np.float32)
    K.check(lib.lspk_d2h(got1.ctypes.data, lib.lspk_tp_window_vector(1), got1.nbytes))
    assert np.array_equal(got1, np.arange(32, dtype=np.float32))
    K.check(lib.lspk_tp_exchange(full.ptr, 0))
    out = np.empty(64, np.float32)
    K.check(lib.lspk_d2h(out.ctypes.data, lib.lspk_tp_window_vector(0), out.nbytes))
    assert np.array_equal(out, np.arange(64, dtype=np.float32) * 0.5)
    assert lib.lspk_tc_check_error() == 0
    K.check(lib.lspk_tp_window_close())
