"""Helpers for the GPU parity tests: device buffers (torch is only the allocator)
and layout shuffles done on the host side of the test."""
import numpy as np
import torch

import darknet_b200 as dn


def dev_nchw(a: np.ndarray):
    """Host NCHW float32 array -> (torch CUDA tensor, dnb_tensor)."""
    t = torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()
    return t, dn.as_tensor(t, dn.NCHW)


def dev_nhwc(a: np.ndarray, dtype=torch.float32):
    """Host NCHW array -> channels-last device tensor with zero padding channels."""
    n, c, h, w = a.shape
    cp = (c + 7) // 8 * 8
    t = torch.zeros((n, h, w, cp), dtype=dtype, device="cuda")
    t[..., :c] = torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda().permute(0, 2, 3, 1).to(dtype)
    return t, dn.as_tensor(t, dn.NHWC, c)


def empty_nchw(n, c, h, w):
    t = torch.full((n, c, h, w), float("nan"), dtype=torch.float32, device="cuda")
    return t, dn.as_tensor(t, dn.NCHW)


def empty_nhwc(n, c, h, w, dtype=torch.float32):
    cp = (c + 7) // 8 * 8
    t = torch.full((n, h, w, cp), float("nan"), dtype=dtype, device="cuda")
    return t, dn.as_tensor(t, dn.NHWC, c)


def host_from_nhwc(t, c) -> np.ndarray:
    """Channels-last device tensor -> host NCHW float32 (padding channels dropped)."""
    return t[..., :c].permute(0, 3, 1, 2).float().contiguous().cpu().numpy()


def padding_is_zero(t, c) -> bool:
    return bool((t[..., c:].float() == 0).all().item()) if t.shape[-1] > c else True


def bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).to(torch.bfloat16).float().numpy()
