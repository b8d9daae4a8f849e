"""logicaffeine_b200 — the Q8 LLM-decode hot path as sm_100a CUDA kernels behind
logicaffeine's native-operator C ABI.  `logicaffeine_b200.llm` is the host-side
mirror of the operator family; `logicaffeine_b200.weights` writes and inspects weight files, `logicaffeine_b200.convert` makes one
from a float checkpoint;
`logicaffeine_b200.build` compiles the library."""

__all__ = ["llm", "weights", "convert", "build"]
