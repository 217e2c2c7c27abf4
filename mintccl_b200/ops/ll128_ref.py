"""NumPy restatement of the LL128 wire format (pack / unpack / validity), used as the CPU oracle.

Wire format (shared with ``csrc/device/proto_ll128.cuh`` and the host simulator): a 128-byte line is
eight 16-byte lane words; lanes 0..6 carry 112 payload bytes, lane 7 carries 8 payload bytes followed by
the 8-byte flag.  Lines come in pairs covering 240 contiguous payload bytes: pair ``p``, half ``h`` holds
payload ``[240p + 128h, +112)`` in lanes 0..6 and ``[240p + 112 + 8h, +8)`` in lane 7.  A warp chunk is
16 lines (1920 payload bytes); line ``(p, h)`` sits at index ``((p // 4) * 2 + h) * 4 + p % 4`` so that
each of the warp's four accesses writes 512 contiguous bytes.

The reference's format (protocol.py:57-100) is the same line with two lines per 8-thread group; there
the flag is the global line index, here it is the FIFO step + 1.
"""
from __future__ import annotations

import numpy as np

LINE, LINE_PAYLOAD, PAIR_PAYLOAD = 128, 120, 240
WARP_LINES, WARP_WIRE, WARP_PAYLOAD = 16, 2048, 1920


def wire_lines(payload: int) -> int:
    pairs, rest = divmod(payload, PAIR_PAYLOAD)
    return pairs * 2 + (0 if rest == 0 else (1 if rest <= LINE_PAYLOAD else 2))


def line_of(pair: int, half: int) -> int:
    return ((pair // 4) * 2 + half) * 4 + pair % 4


def pack(payload: bytes, flag: int) -> np.ndarray:
    """Wire image (uint8, whole warp chunks) of ``payload`` stamped with ``flag``; unused lines stay 0."""
    data = np.frombuffer(bytes(payload), dtype=np.uint8)
    nchunks = max(1, -(-len(data) // WARP_PAYLOAD))
    wire = np.zeros(nchunks * WARP_WIRE, dtype=np.uint8)
    for wc in range(nchunks):
        chunk = data[wc * WARP_PAYLOAD:(wc + 1) * WARP_PAYLOAD]
        nb = len(chunk)
        for li in range(wire_lines(nb)):
            pair, half = divmod(li, 2)
            base = wc * WARP_WIRE + line_of(pair, half) * LINE
            a = chunk[PAIR_PAYLOAD * pair + 128 * half: PAIR_PAYLOAD * pair + 128 * half + 112]
            b = chunk[PAIR_PAYLOAD * pair + 112 + 8 * half: PAIR_PAYLOAD * pair + 112 + 8 * half + 8]
            wire[base: base + len(a)] = a
            wire[base + 112: base + 112 + len(b)] = b
            wire[base + 120: base + 128] = np.frombuffer(np.uint64(flag).tobytes(), dtype=np.uint8)
    return wire


def valid(wire: np.ndarray, nbytes: int, flag: int) -> bool:
    """True when every line that a message of ``nbytes`` needs carries ``flag``."""
    want = np.frombuffer(np.uint64(flag).tobytes(), dtype=np.uint8)
    for wc in range(max(1, -(-nbytes // WARP_PAYLOAD))):
        nb = min(WARP_PAYLOAD, nbytes - wc * WARP_PAYLOAD)
        for li in range(wire_lines(nb)):
            pair, half = divmod(li, 2)
            base = wc * WARP_WIRE + line_of(pair, half) * LINE
            if not np.array_equal(wire[base + 120: base + 128], want):
                return False
    return True


def unpack(wire: np.ndarray, nbytes: int) -> bytes:
    out = np.zeros(nbytes, dtype=np.uint8)
    for wc in range(max(1, -(-nbytes // WARP_PAYLOAD))):
        nb = min(WARP_PAYLOAD, nbytes - wc * WARP_PAYLOAD)
        dst = out[wc * WARP_PAYLOAD: wc * WARP_PAYLOAD + nb]
        for li in range(wire_lines(nb)):
            pair, half = divmod(li, 2)
            base = wc * WARP_WIRE + line_of(pair, half) * LINE
            a0 = PAIR_PAYLOAD * pair + 128 * half
            b0 = PAIR_PAYLOAD * pair + 112 + 8 * half
            la = max(0, min(112, nb - a0))
            lb = max(0, min(8, nb - b0))
            dst[a0:a0 + la] = wire[base: base + la]
            dst[b0:b0 + lb] = wire[base + 112: base + 112 + lb]
    return out.tobytes()


def efficiency() -> float:
    """Payload fraction of the wire: 120 / 128 (2_sendrecv_indirect.py:56 quotes the same 93.75 %)."""
    return LINE_PAYLOAD / LINE
