"""Multi-GPU tests: each case launches one process per GPU with torch.distributed.run over NCCL on 127.0.0.1."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
NGPU = torch.cuda.device_count() if torch.cuda.is_available() else 0


def _run(script, nproc, *args, timeout=600, env=None):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(29500 + nproc), os.path.join(HERE, script), *args]
    e = dict(os.environ)
    e.update(env or {})
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=e)


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_peer_allreduce(nproc):
    if NGPU < nproc:
        pytest.skip(f"needs {nproc} GPUs, found {NGPU}")
    p = _run("mp_peer_allreduce.py", nproc)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "FAILURES 0" in p.stdout


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("nproc", [2, 8])
@pytest.mark.parametrize("mode", ["fused", "nccl"])
def test_tensor_parallel_tiny_model(nproc, mode):
    """TP engine (prefill + graph decode) agrees with the oracle; fused = in-kernel peer-memory all-reduce."""
    if NGPU < nproc:
        pytest.skip(f"needs {nproc} GPUs, found {NGPU}")
    p = _run("mp_tp_model.py", nproc, mode)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "FAILURES 0" in p.stdout


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("nproc", [2, 8])
def test_expert_parallel_tiny_moe(nproc):
    """Expert parallelism over replicated tokens + TP attention with KV heads replicated on rank pairs."""
    if NGPU < nproc:
        pytest.skip(f"needs {nproc} GPUs, found {NGPU}")
    p = _run("mp_tp_model.py", nproc, "fused", "moe")
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "FAILURES 0" in p.stdout


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("nproc", [2, 8])
def test_sequence_parallel_fused_linears(nproc):
    """All-gather->GEMM and GEMM->reduce-scatter kernels over real peer memory (NVLS stores and plain peer stores)."""
    if NGPU < nproc:
        pytest.skip(f"needs {nproc} GPUs, found {NGPU}")
    p = _run("mp_sp_ops.py", nproc)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "FAILURES 0" in p.stdout


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("nproc", [2, 4, 8])
def test_fused_gemm_allreduce_one_trip_and_two_hop(nproc):
    """Decode GEMM + all-reduce in one launch: both tails give the rank-ordered sum of the bf16 partials, the same bits
    on every rank, eagerly and from a replayed CUDA graph."""
    if NGPU < nproc:
        pytest.skip(f"needs {nproc} GPUs, found {NGPU}")
    p = _run("mp_fused_ar.py", nproc)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "FAILURES 0" in p.stdout


@pytest.mark.gpu
@pytest.mark.multigpu(2)
@pytest.mark.parametrize("multicast", ["0", "1"])
@pytest.mark.parametrize("script", ["mp_peer_allreduce.py", "mp_fused_ar.py"])
def test_native_symmetric_heap_backend(script, multicast):
    """The same peer kernels over this package's own heap (virtual-memory blocks shared as POSIX descriptors and
    mapped by every rank) instead of torch's symmetric memory: with peer pointers only, and with its own multicast
    object bound over the blocks (the multimem kernels then run through it)."""
    if NGPU < 2:
        pytest.skip(f"needs 2 GPUs, found {NGPU}")
    p = _run(script, 2, env={"B200RT_SYMM": "native", "B200RT_SYMM_MC": multicast})
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "FAILURES 0" in p.stdout
    assert f"symm backend native multicast {multicast == '1'}" in p.stdout
