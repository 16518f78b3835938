"""Helpers of the Tanolorn tests: device tensors in the dtypes the engine binds (small tables float32, matrices bfloat16 or float32)."""
import numpy as np
import torch

TABLE_ENDINGS = ("norm1", "norm2", "final.norm", ".norm", ".b", ".conv", ".dt_bias", ".A_log", ".D", ".router", ".correction")


def is_table(name: str) -> bool:
    return name.endswith(TABLE_ENDINGS)


def device_tensors(W: dict, exact: bool):
    out = {}
    for name, a in W.items():
        t = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()
        out[name] = t if (exact or is_table(name)) else t.to(torch.bfloat16)
    return out
