"""Helpers shared by the GPU parity tests (device tensors from host numpy, tolerances)."""
import numpy as np
import torch

# Tolerances of the parity tests: bf16 outputs within 2e-2 max-abs and 1e-2 relative of the f32 reference; f32 within 1e-4.
BF16_ABS = 2e-2
BF16_REL = 1e-2
F32_ABS = 1e-4


def dev(array: np.ndarray, dtype=None) -> torch.Tensor:
    tensor = torch.from_numpy(np.ascontiguousarray(array))
    if dtype is not None:
        tensor = tensor.to(dtype)
    return tensor.cuda()


def dev_u32(array: np.ndarray) -> torch.Tensor:
    """uint32 host array as an int32-typed device buffer with the same bits."""
    return torch.from_numpy(np.ascontiguousarray(array, dtype=np.uint32).view(np.int32)).cuda()


def host(tensor: torch.Tensor) -> np.ndarray:
    return tensor.detach().float().cpu().numpy()


def assert_close_bf16(actual: np.ndarray, expected: np.ndarray, what: str):
    error = np.abs(actual.astype(np.float64) - expected.astype(np.float64))
    worst = float(error.max()) if error.size else 0.0
    bound = BF16_ABS + BF16_REL * np.abs(expected)
    bad = int((error > bound).sum())
    assert bad == 0 and worst <= BF16_ABS + BF16_REL * float(np.abs(expected).max()), (
        f"{what}: max abs err {worst:.3e}, {bad} of {error.size} outside {BF16_ABS}+{BF16_REL}*|ref|; "
        f"first bad index {np.argwhere(error > bound)[:3].tolist()}")


def assert_close_f32(actual: np.ndarray, expected: np.ndarray, what: str, tolerance: float = F32_ABS):
    error = np.abs(actual.astype(np.float64) - expected.astype(np.float64))
    worst = float(error.max()) if error.size else 0.0
    assert worst <= tolerance, f"{what}: max abs err {worst:.3e} > {tolerance}; at {np.unravel_index(error.argmax(), error.shape)}"
