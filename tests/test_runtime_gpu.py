"""The rank runtime under the engine: the host thread sits beside its GPU and the long-lived buffers come from the
rank's HBM arena (the GPU form of the reference's pinned workers over node-local arenas,
test_linux_threading.mojo:104-136, 217-302)."""
import pytest
import torch

from mojo_linuxperiments_b200.models import config as C

pytestmark = pytest.mark.gpu


def test_engine_buffers_live_in_the_rank_arena_and_the_thread_beside_its_gpu():
    from mojo_linuxperiments_b200 import hostrt
    from mojo_linuxperiments_b200.engine.engine import Engine
    from mojo_linuxperiments_b200.models.decoder import KVState
    cfg = C.tiny_dense()
    rt = C.RuntimeConfig(max_seq_len=128)
    saved = hostrt.get_thread_affinity()
    try:
        eng = Engine(cfg, rt, seed=0)
        eng.start_batch(3, 64)
        run = eng.runtime
        assert run.arena is not None, run.notes
        # the KV cache, its page table and the sequence lengths are carved from the arena, in that order
        assert run.owns(eng.kv.storage) and run.owns(eng.kv.page_table) and run.owns(eng.kv.seq_lens)
        need = KVState.nbytes(cfg, rt, 3, rt.max_seq_len)
        rep = eng.memory_report()
        assert rep["kv_arena"]["placement_ok"]
        assert rep["kv_arena"]["used"] >= need - 3 * 1024 and rep["kv_arena"]["high_water"] == rep["kv_arena"]["used"]
        assert rep["kv_arena"]["remaining"] == rep["kv_arena"]["size"] - rep["kv_arena"]["used"]
        # and the model still decodes out of it
        prompts = torch.randint(0, cfg.vocab, (3, 20), generator=torch.Generator().manual_seed(0))
        out = eng.generate(prompts, 4)
        assert out.shape == (3, 4)
        assert run.owns(eng.kv.storage)
        # a bigger batch replaces the arena; the old one goes when its last tensor does
        eng.start_batch(5, 64)
        assert run.owns(eng.kv.storage) and eng.memory_report()["kv_arena"]["used"] >= KVState.nbytes(cfg, rt, 5, rt.max_seq_len) - 3 * 1024
        if run.numa_node < 0 or not run.pinned_cpus:
            pytest.skip(f"no NUMA node reported for this GPU / not pinned: {run.notes}")
        cpu, node = hostrt.get_current_cpu_and_node()
        assert node == run.numa_node and cpu in run.pinned_cpus
        assert rep["host_thread"]["numa_node"] == run.numa_node
    finally:
        hostrt.set_thread_affinity(saved)
