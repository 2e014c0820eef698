"""Block-format facts (pure Python, no GPU): sizes as in include/ttq.h."""
from ._lib import FMT_Q4_K, FMT_Q6_K, FMT_Q8_0, FMT_TQ3

BLOCK_ELEMS = {FMT_Q8_0: 32, FMT_Q4_K: 256, FMT_Q6_K: 256}
BLOCK_BYTES = {FMT_Q8_0: 34, FMT_Q4_K: 144, FMT_Q6_K: 210}
FORMAT_NAMES = {FMT_Q8_0: "Q8_0", FMT_Q4_K: "Q4_K", FMT_Q6_K: "Q6_K", FMT_TQ3: "TQ3"}


def packed_bytes(fmt: int, n: int, k: int) -> int:
    """Canonical byte count of an [n][k] matrix = algorithmic weight bytes of one forward."""
    if fmt == FMT_TQ3:
        if n % 128 or k % 128:
            raise ValueError("the trellis format needs N and K in multiples of 128")
        return n * k * 3 // 8 + 2 * n + k // 8
    if k % BLOCK_ELEMS[fmt]:
        raise ValueError(f"K={k} is not a multiple of the {FORMAT_NAMES[fmt]} block length")
    return n * (k // BLOCK_ELEMS[fmt]) * BLOCK_BYTES[fmt]
