"""GPU test of the tensor-parallel decode engine: 2 ranks on 2 GPUs (NCCL all-reduce after each
row-parallel layer), logits of every rank against a distributed fp32 torch forward of the same
sharded network; tolerance max-rel 1e-2.  Skipped where fewer than 2 GPUs are visible."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mode,chain", [("nccl", "fused"), ("peer", "fused"), ("peer", "unfused"), ("peer", "glued"), ("nccl", "glued")])
def test_tensor_parallel_decode_world2(mode, chain):
    """mode nccl: NCCL all-reduce after each row-parallel layer; mode peer: the fused transform + all-reduce +
    residual kernel over NVLink peer memory (plain peer stores; NVLS is off in both).  chain: the short
    tensor-parallel chain (fused glue kernels), the 15-launch one, or the one with the norms inside the matvecs."""
    port = 29600 + os.getpid() % 1000 + (0 if mode == "nccl" else 1) + {"fused": 0, "unfused": 2, "glued": 4}[chain]
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), str(r), "2", str(port), mode, chain],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=240)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append("timed out\n" + p.communicate()[0])
    for p, out in zip(procs, outs):
        assert p.returncode == 0, out[-2000:]
