"""The e4m3 codes of the prompt GEMM's operands against torch's float8_e4m3fn decoder (CPU only): every code stands for the
integer it was made from, and the two parts of every 8-bit value add up to it."""
import torch

from spy_b200 import quants


def _decode(code: int) -> float:
    return float(torch.tensor([code], dtype=torch.uint8).view(torch.float8_e4m3fn).float()[0])


def test_small_integers_are_exact():
    for v in range(16):
        assert _decode(quants.e4m3_of_small(v)) == float(v)
    for v in range(-15, 16):
        assert _decode(quants.e4m3_of_signed(v)) == float(v)


def test_every_byte_is_the_sum_of_its_two_parts():
    for y in range(-128, 128):
        hi, lo = quants.e4m3_split(y)
        assert 0 <= hi <= 0xFF and 0 <= lo <= 0x57
        assert _decode(hi) + _decode(lo) == float(y)
        assert _decode(hi) % 16 == 0 and 0 <= _decode(lo) <= 15
