"""Helpers of the Savidra tests: device tensors in the dtypes the engine binds (vectors and small tables float32, matrices bfloat16 or float32)."""
import numpy as np
import torch

TABLE_ENDINGS = (".conv", ".talk")


def is_table(name: str, a) -> bool:
    return np.ndim(a) < 2 or name.endswith(TABLE_ENDINGS)


def device_tensors(W: dict, exact: bool):
    out = {}
    for name, a in W.items():
        t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
        out[name] = t if (exact or is_table(name, a)) else t.to(torch.bfloat16)
    return out
