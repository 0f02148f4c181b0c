"""Host-resident lookup tables: plain and node-shared (one mmap per node under a shared directory).
Reference tests: tests/engine/backends/fsdp2/test_dcp_node_shared.py and the qwen4_exp table tests."""
import os

import torch

from dist_utils import run_distributed
from torchturbo_b200.models.modules.cpu_resident import CPUResidentParameter, NodeSharedCPUResidentParameter


def test_plain_table_lookup_stays_on_host_and_out_of_state():
    tab = CPUResidentParameter(50, 8, dtype=torch.float32, pin=False)
    rows = torch.arange(50 * 8, dtype=torch.float32).view(50, 8)
    tab.load_rows(0, rows[:30])
    tab.load_rows(30, rows[30:])
    idx = torch.tensor([[3, 49], [0, 3]])
    out = tab(idx)
    assert out.shape == (2, 2, 8) and torch.equal(out, rows[idx])
    parent = torch.nn.Sequential(torch.nn.Linear(4, 4))
    parent.tab = tab
    parent.to(torch.float64)                       # dtype / device moves of the parent leave the table alone
    assert tab.table.dtype == torch.float32 and tab.table.device.type == "cpu"
    assert not any(k.startswith("tab") for k in parent.state_dict())
    assert not any(True for _ in tab.parameters())  # frozen: invisible to optimizers and to FSDP


def _w_node_shared(rank, world, shm_dir):
    import torch.distributed as dist

    tab = NodeSharedCPUResidentParameter(64, 4, dtype=torch.bfloat16, name="ple", local_rank=rank, shm_dir=shm_dir)
    assert os.path.exists(tab.path)
    full = (torch.arange(64 * 4, dtype=torch.float32).view(64, 4) / 7).bfloat16()
    # every rank offers rows; only the node's first rank writes them into the shared file
    tab.load_rows(0, full[:40] if rank == 0 else torch.zeros(40, 4))
    tab.load_rows(40, full[40:] if rank == 0 else torch.zeros(24, 4))
    tab.finish_loading()
    idx = torch.tensor([0, 63, 17 + rank])
    assert torch.equal(tab(idx), full[idx]), f"rank {rank} does not see the rows the writer stored"
    n_files = len([f for f in os.listdir(shm_dir) if f.startswith("ttb200_ple_")])
    assert n_files == 1, "one mapping per node, not one per rank"
    dist.barrier()
    tab.close()
    dist.barrier()
    assert not os.path.exists(tab.path)


def test_node_shared_table_is_written_once_and_read_by_all_ranks(tmp_path):
    run_distributed(_w_node_shared, 3, str(tmp_path))
