"""The reference's random numbers: XorShift64 with shifts 13, 7, 17 and a
24-bit float (tools/infer/src/main.rs:1025-1045), and the per-session seed
mix of its engine (crates/cellm-sdk/src/lib.rs:526-535)."""
from __future__ import annotations

_M = 0xFFFFFFFFFFFFFFFF


class XorShift64:
    def __init__(self, seed: int):
        self.state = max(int(seed) & _M, 1)

    def next_u64(self) -> int:
        x = self.state
        x ^= (x << 13) & _M
        x ^= x >> 7
        x ^= (x << 17) & _M
        self.state = x
        return x

    def next_f32(self) -> float:
        return float(self.next_u64() >> 40) / float(1 << 24)


def session_seed(session: int, seed: int) -> int:
    x = (int(session) ^ 0x9E3779B97F4A7C15) & _M
    x = (x * 0xBF58476D1CE4E5B9) & _M
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _M
    x ^= x >> 31
    return (x ^ int(seed)) & _M
