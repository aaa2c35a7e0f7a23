"""CPU oracle of the GGUF quantized-matmul path -- test infrastructure, never a product path.

Only tests/, the smoke check and the CPU-baseline / reference arms of the benchmark may
import this package.  ``oracle.cpu`` wraps the C restatement (gguf_oracle.c);
``oracle.build_ref`` builds the reference plugin's own CUDA extension for GPU parity runs.
"""

import os
from pathlib import Path


def reference_root():
    """Where the reference plugin's checkout lies, or None: the directory named by the
    GGUF_REFERENCE_ROOT environment variable, else a directory called ``reference`` next to this
    repository.  Everything that reads the reference (building its CUDA extension, regenerating
    fixtures, comparing tables) goes through here and skips when the answer is None."""
    cands = []
    if os.environ.get("GGUF_REFERENCE_ROOT"):
        cands.append(Path(os.environ["GGUF_REFERENCE_ROOT"]))
    cands.append(Path(__file__).resolve().parent.parent.parent / "reference")
    for c in cands:
        if (c / "vllm_gguf_plugin").is_dir():
            return c
    return None
