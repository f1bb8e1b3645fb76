"""The attention calls of one denoise step (8 double-stream + 24 single-stream blocks, and the
doubled sequence under classifier-free guidance) issued one by one and as one CUDA graph: the
replayed graph must reproduce the eager calls bit for bit, and a call of each kind is held
against the ideal oracle. Mirrors the reference's per-step loop
(src/backend/cuda/flux_transformer.cu:412-439, tools/serve.cu:563-566)."""
import numpy as np
import pytest

from tests._util import assert_parity, dev_bf16, host_bits, host_f32

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("guidance", [False, True])
def test_graph_replay_equals_eager_calls(orc, guidance):
    import torch
    assert torch.cuda.is_available()
    import f2k_cuda_b200 as f2k
    from f2k_cuda_b200.inputs import Workload, make_problem, token_positions
    from f2k_cuda_b200.step import DoubleCall, SingleCall, StepAttention
    B, St, grid, H, D = 1, 64, (12, 16), 4, 128
    w = Workload("step", B, St, (grid,), n_heads=H, seed=0x57E9)
    Si, S = w.seq_img, w.seq
    pt, pi = token_positions(w)
    tabs = (*f2k.build_rope_4axis_tables((32,) * 4, pt, 2000.0), *f2k.build_rope_4axis_tables((32,) * 4, pi, 2000.0))
    dtab = [torch.from_numpy(t).cuda() for t in tabs]
    dtab_c = [torch.cat([dtab[0], dtab[2]]).contiguous(), torch.cat([dtab[1], dtab[3]]).contiguous()]
    gammas = make_problem(w).gammas
    dg = [dev_bf16(g) for g in gammas]
    gen = torch.Generator(device="cuda").manual_seed(0x57E9)
    rnd = lambda n: torch.randn(B, n, H, D, device="cuda", generator=gen).to(torch.bfloat16)  # noqa: E731
    nan = lambda n: torch.full((B, n, H, D), float("nan"), device="cuda", dtype=torch.bfloat16)  # noqa: E731

    def model_pass():
        return ([DoubleCall(rnd(St), rnd(St), rnd(St), rnd(Si), rnd(Si), rnd(Si), nan(St), nan(Si)) for _ in range(8)],
                [SingleCall(rnd(S), rnd(S), rnd(S), nan(S)) for _ in range(24)])

    passes = [model_pass() for _ in range(2 if guidance else 1)]      # conditional, unconditional
    step = StepAttention(B, St, Si, H, D)
    assert step.ok(), step.last_error()
    outs = [t for dbl, sgl in passes for c in dbl for t in (c.o_txt, c.o_img)] + [c.o for _, sgl in passes for c in sgl]

    assert step.run(passes, dg, dtab, dtab_c) == (64 if guidance else 32)
    torch.cuda.synchronize()
    assert step.device_status() == 0
    eager = [o.clone() for o in outs]
    assert all(bool(torch.isfinite(o).all()) for o in eager)

    graph, calls = step.capture(passes, dg, dtab, dtab_c)
    assert calls == (64 if guidance else 32)
    for o in outs:
        o.fill_(float("nan"))
    graph.replay()
    torch.cuda.synchronize()
    assert step.device_status() == 0
    for i, (a, b) in enumerate(zip(eager, outs)):
        assert torch.equal(a, b), f"output {i} of the replayed graph differs from the eager call"
    graph.replay()                                   # and again: the graph holds no state
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(eager, outs))

    # one call of each kind, of the last pass, against fp32/double host math
    dbl, sgl = passes[-1]
    c = dbl[3]
    r_t, r_i = orc.joint_path(q_txt=host_bits(c.q_txt), k_txt=host_bits(c.k_txt), v_txt=host_bits(c.v_txt),
                              q_img=host_bits(c.q_img), k_img=host_bits(c.k_img), v_img=host_bits(c.v_img),
                              gammas=gammas, tables=tabs, eps=1e-6)
    assert_parity(host_f32(c.o_txt), r_t, "double-stream call, text rows")
    assert_parity(host_f32(c.o_img), r_i, "double-stream call, image rows")
    s = sgl[11]
    tabs_c = (np.concatenate([tabs[0], tabs[2]]), np.concatenate([tabs[1], tabs[3]]))
    _, r = orc.joint_path(q_img=host_bits(s.q), k_img=host_bits(s.k), v_img=host_bits(s.v),
                          gammas=(None, None, gammas[2], gammas[3]), tables=(None, None, *tabs_c), eps=1e-6)
    assert_parity(host_f32(s.o), r, "single-stream call")
