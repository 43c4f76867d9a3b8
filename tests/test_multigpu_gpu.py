"""Multi-GPU paths on real GPUs (skipped when fewer than two are visible).

Each test launches one process per GPU with torchrun-style environment
variables on 127.0.0.1 and checks the sharded result against the oracle.
"""

import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

WORKER = r'''
import math, os, sys
sys.path.insert(0, os.environ["TF_ROOT"])
import torch, torch.distributed as dist
from oracle import attention_oracle as orc
from tilefusion_b200.shard import ShardedDecoder, kv_slice, prefill_sharded, head_slice

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
# decode sharded by KV length: every rank must end with the full answer
b, h, lk, d = 2, 4, 6000, 128
q, k, v = orc.seeded_inputs(51, (b, h, 1, d), (b, h, lk, d), (b, h, lk, d), 1.0)
k0, k1 = kv_slice(lk, rank, world)
ref, lse_ref = orc.decode_fp32(q, k, v)
qd, kd, vd = q.to(dev), k[:, :, k0:k1].contiguous().to(dev), v[:, :, k0:k1].contiguous().to(dev)
for transport in ("p2p", "nccl"):
    dec = ShardedDecoder(b, h, d, torch.float16, dev, transport=transport)
    assert dec.transport == transport, (transport, getattr(dec, "transport_fallback_reason", ""))
    for _ in range(5):      # several steps: gather areas and flags are reused between steps
        o, lse = dec(qd, kd, vd)
    assert orc.max_abs(o.cpu(), ref) <= 2e-2 and orc.rel_l2(o.cpu(), ref) <= 1e-3, "decode O " + transport
    assert orc.max_abs(lse.cpu(), lse_ref) <= 1e-3, "decode LSE " + transport
    torch.cuda.synchronize()
    dist.barrier()
# prefill sharded by heads: no collective
n, l = 12, 384
q2, k2, v2 = orc.seeded_inputs(52, (n, l, d), (n, l, d), (n, l, d), 0.5)
out, (h0, h1) = prefill_sharded(q2.to(dev), k2.to(dev), v2.to(dev), 1.0 / math.sqrt(d))
ref2, _ = orc.attention_fp32(q2[h0:h1], k2[h0:h1], v2[h0:h1], 1.0 / math.sqrt(d))
assert (h0, h1) == head_slice(n, rank, world)
assert orc.max_abs(out.cpu(), ref2) <= 2e-2 and orc.rel_l2(out.cpu(), ref2) <= 1e-3, "prefill"
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_decode_and_prefill(world, tmp_path):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), TF_ROOT=str(ROOT))
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"rank {r} ok" in out, out[-2000:]
