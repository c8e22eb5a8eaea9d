"""Helpers shared by the GPU tests: run the CUDA engine through the C ABI
(ctypes, via the package's calculator) and bring the result to numpy."""

import numpy as np


def gpu_compute(points, box, periodic, cutoff, full, quantities="ijSdD", algorithm="auto", sorted=False, calculator=None):
    import torch

    import vesin_b200

    device = torch.device("cuda", 0)
    if calculator is None:
        calculator = vesin_b200.NeighborList(cutoff=cutoff, full_list=full, algorithm=algorithm, sorted=sorted)
    outputs = calculator.compute(
        torch.tensor(np.asarray(points, dtype=np.float64).reshape(-1, 3), device=device),
        torch.tensor(np.asarray(box, dtype=np.float64), device=device),
        torch.tensor(np.asarray(periodic, dtype=bool), device=device),
        quantities,
        copy=False,
    )
    result = {}
    for key, value in zip(quantities, outputs):
        value = value.cpu().numpy()
        if key in "ij":
            value = value.astype(np.int64)
        result[key] = value
    return result
