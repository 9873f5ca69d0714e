"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

from oracle import cpu_oracle as o

TORCH_DTYPE = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
# north_star tolerances: FP32 max-abs 1e-4 and relative L2 1e-5; FP16/BF16 max-abs 2e-2 vs the FP32 reference
TOL_F32_ABS, TOL_F32_REL_L2, TOL_16_ABS = 1e-4, 1e-5, 2e-2


def payload_to_torch(a: np.ndarray, dtype: str) -> torch.Tensor:
    """uint16 payloads (or float32) -> torch tensor of `dtype` sharing the bit pattern."""
    if dtype == "f32":
        return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32))
    t = torch.from_numpy(np.ascontiguousarray(a).view(np.int16))
    return t.view(TORCH_DTYPE[dtype])


def torch_to_f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def rounded_inputs(shape, dtype: str, seed: int, scale: float = 1.0, n: int = 3):
    """n N(0,1)*scale tensors rounded to `dtype`: (float32 values as the oracle sees them, torch tensors)."""
    rng = np.random.default_rng(seed)
    vals, tens = [], []
    for _ in range(n):
        x = (rng.standard_normal(shape) * scale).astype(np.float32)
        p = o.round_to(x, dtype)
        vals.append(o.widen(p, dtype))
        tens.append(payload_to_torch(p, dtype))
    return vals, tens


def assert_close(got: np.ndarray, want: np.ndarray, dtype: str, what: str = ""):
    assert np.all(np.isfinite(got)), f"{what}: non-finite output"
    err = np.abs(got.astype(np.float64) - want.astype(np.float64)).max()
    if dtype == "f32":
        rel = np.linalg.norm((got - want).astype(np.float64)) / max(np.linalg.norm(want.astype(np.float64)), 1e-30)
        assert err <= TOL_F32_ABS and rel <= TOL_F32_REL_L2, f"{what}: max-abs {err:.3e} rel-L2 {rel:.3e}"
    else:
        assert err <= TOL_16_ABS, f"{what}: max-abs {err:.3e}"
