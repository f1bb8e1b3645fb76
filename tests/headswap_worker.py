"""Child process of tests/test_headswap_gpu.py::test_one_process_per_gpu (one per GPU, under
torchrun): sequence-parallel attention by head exchange over CUDA IPC against the CPU oracle."""
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
    import f2k_cuda_b200 as f2k
    from f2k_cuda_b200.headswap import HeadExchangeAttention
    from f2k_cuda_b200.inputs import Workload, make_problem
    from tests._util import assert_parity, dev_bf16, host_f32
    per, H, D = 264, 8, 128                      # 264 = 2 tiles + 8 tokens: every shard ends in a ragged tile
    S = world * per
    w = Workload("hx", 1, 0, ((world * 8, 33),), seed=0x1DD)
    p = make_problem(w, heads=H)                 # every rank draws the same full problem (small)
    cos, sin = f2k.build_rope_4axis_tables((32,) * 4, p.pos_img, 2000.0)
    sl = slice(rank * per, (rank + 1) * per)
    hx = HeadExchangeAttention(per, H, D, world, rank)
    assert hx.ok(), hx.last_error()
    assert hx.attach_distributed(), hx.last_error()
    q, k, v = (dev_bf16(np.ascontiguousarray(x[:, sl])) for x in (p.q_img, p.k_img, p.v_img))
    gq, gk = dev_bf16(p.gammas[2]), dev_bf16(p.gammas[3])
    dcos, dsin = torch.from_numpy(cos[sl].copy()).cuda(), torch.from_numpy(sin[sl].copy()).cuda()
    # the oracle first: computed between two steps it would put seconds of skew between the ranks,
    # which the next step's device-side waits would have to absorb
    _, ref = oracle.load_oracle().joint_path(q_img=p.q_img, k_img=p.k_img, v_img=p.v_img,
                                             gammas=(None, None, p.gammas[2], p.gammas[3]),
                                             tables=(None, None, cos, sin), eps=1e-6)
    dist.barrier()
    # back to back: no collective, no host synchronisation between steps. Steps 0-3 run the exchange
    # as a kernel of its own, steps 4-7 inside the attention kernel (the fused form), steps 8-11 with
    # the copy engines under the attention kernel.
    for step in range(12):
        if step < 4:
            assert hx.exchange_in(q, k, v, gq, gk, dcos, dsin, 1e-6), hx.last_error()
            assert hx.attend(), hx.last_error()
        elif step < 8:
            assert hx.forward(q, k, v, gq, gk, dcos, dsin, 1e-6), hx.last_error()
        else:
            assert hx.exchange_in_copy(q, k, v, gq, gk, dcos, dsin, 1e-6), hx.last_error()
            assert hx.attend(), hx.last_error()
        o = hx.output()
        assert o is not None, hx.last_error()
        got = o.clone()                          # stream order: after the waits of output()
        if step in (0, 3, 4, 7, 8, 11):
            torch.cuda.synchronize()
            assert hx.device_status() == 0, hx.last_error()
            assert_parity(host_f32(got), ref[:, sl], f"rank {rank} step {step}")
    dist.barrier()
    if rank == 0:
        print("HEADSWAP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
