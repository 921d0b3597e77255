"""Device-side helpers of the GPU tests (torch is used for memory and streams only)."""
import numpy as np
import torch

AD = 256


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def pos_tensor(p):
    return torch.tensor([int(p)], dtype=torch.int32, device="cuda")


def poisoned_cache(q27, orc_cache, nkvh, n_ctx, n, q8=True):
    """Uploads an oracle-built cache and fills every row >= n with 0xFF bytes (NaN scales / values):
    nothing past the end of the sequence may influence a result."""
    c = np.array(orc_cache, copy=True)
    if q8:
        vals = c[: nkvh * n_ctx * AD].reshape(nkvh, n_ctx, AD)
        sc = c[nkvh * n_ctx * AD:].reshape(nkvh, n_ctx, 16)
        vals[:, n:] = 0x7F
        sc[:, n:] = 0xFF
    else:
        c.reshape(nkvh, n_ctx, AD * 2)[:, n:] = 0xFF
    return torch.from_numpy(c).cuda()
