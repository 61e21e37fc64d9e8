"""Raw tensor files and a command-line checker, for workflows that exchange ``.bin`` files.

Counterparts of the reference's ``tensor_to_file`` / ``tensor_from_file``
(examples/utils/utils.py:20-42; bf16 travels as 16-bit integers) and of its result checker
(examples/utils/verify_result.py:137-149). Unlike the reference's checker, a failed
comparison exits non-zero.

    python -m mm_rs_with_catlass_b200.utils.io out.bin golden.bin bf16 M N K
"""
from __future__ import annotations

import sys

import numpy as np
import torch

_NAMES = {"fp32": torch.float32, "float": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16,
          "int8": torch.int8, "int32": torch.int32}


def tensor_to_file(t: torch.Tensor, path: str) -> None:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        t.view(torch.int16).numpy().tofile(path)
    else:
        t.numpy().tofile(path)


def tensor_from_file(path: str, dtype: torch.dtype, shape=None) -> torch.Tensor:
    if dtype == torch.bfloat16:
        t = torch.from_numpy(np.fromfile(path, dtype=np.int16)).view(torch.bfloat16)
    else:
        np_dt = {torch.float32: np.float32, torch.float16: np.float16, torch.int8: np.int8, torch.int32: np.int32}[dtype]
        t = torch.from_numpy(np.fromfile(path, dtype=np_dt))
    return t.reshape(shape) if shape is not None else t


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 6:
        print(__doc__)
        return 2
    from .verify import verify
    out_path, gold_path, dt, m, n, k = argv
    dtype = _NAMES[dt]
    out = tensor_from_file(out_path, dtype, (int(m), int(n)))
    gold = tensor_from_file(gold_path, torch.float32, (int(m), int(n)))
    r = verify(out, gold, int(k), dtype)
    print(r)
    return 0 if r.ok else 1


if __name__ == "__main__":
    sys.exit(main())
