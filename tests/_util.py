"""Helpers shared by the tests: error metrics, host<->device moves, reference-style inputs."""
import numpy as np

# The parity gate of this path: bf16 output against fp32/double host math.
MAX_ABS_TOL = 2e-2
COSINE_TOL = 0.9999


def metrics(got: np.ndarray, ref: np.ndarray):
    a = np.asarray(got, np.float64).ravel()
    b = np.asarray(ref, np.float64).ravel()
    max_abs = float(np.max(np.abs(a - b))) if a.size else 0.0
    cos = float(a @ b / np.sqrt((a @ a) * (b @ b) + 1e-300)) if a.size else 1.0
    rel = float(np.sqrt(((a - b) ** 2).sum() / ((b * b).sum() + 1e-300))) if a.size else 0.0
    return max_abs, cos, rel


def assert_parity(got, ref, what="", max_abs_tol=MAX_ABS_TOL, cos_tol=COSINE_TOL):
    max_abs, cos, rel = metrics(got, ref)
    assert np.isfinite(np.asarray(got, np.float64)).all(), f"{what}: non-finite output"
    assert max_abs <= max_abs_tol and cos >= cos_tol, \
        f"{what}: max_abs={max_abs:.4g} (tol {max_abs_tol}) cos={cos:.6f} (tol {cos_tol}) rel={rel:.4g}"
    return max_abs, cos, rel


def dev_bf16(bits: np.ndarray):
    """uint16 bf16 bit patterns -> torch.bfloat16 tensor on cuda:0."""
    import torch
    return torch.from_numpy(np.ascontiguousarray(bits).view(np.int16)).view(torch.bfloat16).cuda()


def host_bits(t) -> np.ndarray:
    """torch.bfloat16 tensor -> uint16 bit patterns."""
    import torch
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def host_f32(t) -> np.ndarray:
    from f2k_cuda_b200.inputs import from_bf16_bits
    return from_bf16_bits(host_bits(t))


def uniform_bits(seed, stream, shape):
    """U(-0.5, 0.5) rounded to bf16: the distribution of the reference's attention tests
    (F2K_CUDA tests/test_attention.cu:21-27)."""
    from f2k_cuda_b200.inputs import to_bf16_bits, uniform01
    n = int(np.prod(shape))
    return to_bf16_bits((uniform01(seed, stream, n) - 0.5).astype(np.float32)).reshape(shape)


def normal_bits(seed, stream, shape):
    from f2k_cuda_b200.inputs import normal, to_bf16_bits
    return to_bf16_bits(normal(seed, stream, int(np.prod(shape)))).reshape(shape)
