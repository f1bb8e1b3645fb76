"""Child process of tests/test_seqpar_gpu.py::test_one_process_per_gpu (one per GPU, under
torchrun): sequence-parallel attention over CUDA IPC + NCCL against the CPU oracle."""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import oracle
    from f2k_cuda_b200.seqpar import SequenceParallelAttention, shard_bounds
    from tests._util import assert_parity, dev_bf16, host_f32, normal_bits
    B, per, H, D = 1, 264, 4, 128               # 264 = 2 tiles + 8 keys: every shard ends in a ragged tile
    S = world * per
    q, k, v = (normal_bits(0x1DC, i, (B, S, H, D)) for i in range(3))
    b, e = shard_bounds(S, world, rank)
    sp = SequenceParallelAttention(B, per, H, D, world, rank)
    assert sp.ok(), sp.last_error()
    assert sp.attach_distributed(), sp.last_error()
    dq = dev_bf16(q[:, b:e])
    _, ref = oracle.load_oracle().joint_path(q_img=q, k_img=k, v_img=v)   # before the steps: no skew between them
    dist.barrier()
    # (overlap, head groups a slot is pulled in; 0 = the library's choice)
    for step, (overlap, groups) in enumerate(((True, 0), (False, 0), (True, 2), (True, 0), (True, 4))):
        if groups:
            os.environ["F2K_SEQPAR_GROUPS"] = str(groups)
        else:
            os.environ.pop("F2K_SEQPAR_GROUPS", None)
        ks, vs = sp.local_kv()
        ks.copy_(dev_bf16(k[:, b:e])); vs.copy_(dev_bf16(v[:, b:e]))
        # no collective here: readiness travels as words in the shard buffers
        do = torch.full_like(dq, float("nan"))
        assert sp.forward(dq, do, overlap=overlap), sp.last_error()
        torch.cuda.synchronize()
        assert sp.device_status() == 0, sp.last_error()
        assert_parity(host_f32(do), ref[:, b:e], f"rank {rank} step {step}")
    dist.barrier()
    if rank == 0:
        print("SEQPAR_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
