"""Guard bands for device outputs.

compute-sanitizer is not available to these tests, so an edge tile that stores
one row or sixteen bytes past the end of an output would go unnoticed with an
exact-size allocation.  ``Guarded`` places the output in the middle of a larger
allocation whose 4 KiB on both sides hold a 0x5A pattern, hands out the view in
between, and checks afterwards that both bands are untouched.  The payload
itself is pre-filled with 0xA5 so that elements a kernel forgot to write show
up as well (``unwritten()``).
"""
import numpy as np

BAND = 4096
PATTERN = 0x5A
FILL = 0xA5


class Guarded:
    def __init__(self, torch, shape, dtype, align=16, offset=0):
        """`offset` bytes shift the payload off its natural alignment (for the
        unaligned-pointer paths); the payload start is `align`-aligned otherwise."""
        self.torch = torch
        elem = torch.empty((), dtype=dtype).element_size()
        self.nbytes = int(np.prod(shape)) * elem
        raw = torch.full((BAND + self.nbytes + BAND + 2 * align,), PATTERN, dtype=torch.uint8, device="cuda")
        base = raw.data_ptr() + BAND
        start = BAND + (-base) % align + offset
        assert offset % elem == 0
        self.raw, self.start = raw, start
        raw[start:start + self.nbytes] = FILL
        self.view = raw[start:start + self.nbytes].view(dtype).view(shape)

    def bands_intact(self) -> bool:
        lo = self.raw[:self.start]
        hi = self.raw[self.start + self.nbytes:]
        return bool((lo == PATTERN).all()) and bool((hi == PATTERN).all())

    def unwritten(self) -> int:
        """Bytes of the payload that still hold the pre-fill pattern in runs of a
        whole element (a legitimately computed 0xA5 byte is possible for int8
        outputs, so callers compare with a small allowance there)."""
        return int((self.raw[self.start:self.start + self.nbytes] == FILL).sum())
