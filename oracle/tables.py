"""Chess-geometry tables of the lc0 policy encoding, generated from first principles.

The reference ships these as literal arrays (neural/encoder.cc:339 move
strings, neural/tables/attention_policy_map.h:24 and :386,
neural/tables/policy_map.h:24); here they are derived from the rules that
define them, and the host-only tests compare every entry with the reference's
arrays when the reference tree is available.

Square index = rank * 8 + file (a1 = 0 ... h8 = 63).
"""
import functools

import numpy as np

NUM_MOVES = 1858
_KNIGHT = ((1, 2), (2, 1), (2, -1), (1, -2), (-1, -2), (-2, -1), (-2, 1), (-1, 2))
# Direction order of the 56 queen-move planes of the convolutional policy head.
_QUEEN_DIRS = ((0, 1), (1, 1), (1, 0), (1, -1), (0, -1), (-1, -1), (-1, 0), (-1, 1))


def _name(sq):
    return "abcdefgh"[sq % 8] + str(sq // 8 + 1)


def _reachable(a, b):
    """True when a queen or a knight standing on `a` attacks `b` on an empty board."""
    if a == b:
        return False
    dx, dy = b % 8 - a % 8, b // 8 - a // 8
    if dx == 0 or dy == 0 or abs(dx) == abs(dy):
        return True
    return (abs(dx), abs(dy)) in ((1, 2), (2, 1))


@functools.lru_cache(None)
def move_strings():
    """The 1858 policy moves in index order: for every from-square the reachable
    to-squares in ascending order, then the 66 under/queen promotions
    (file a..h, capture-left / push / capture-right, q r b)."""
    moves = [_name(a) + _name(b) for a in range(64) for b in range(64) if _reachable(a, b)]
    for f in range(8):
        for t in (f - 1, f, f + 1):
            if 0 <= t < 8:
                for piece in "qrb":
                    moves.append(_name(48 + f) + _name(56 + t) + piece)
    assert len(moves) == NUM_MOVES
    return tuple(moves)


@functools.lru_cache(None)
def _move_index():
    return {m: i for i, m in enumerate(move_strings())}


@functools.lru_cache(None)
def attn_policy_map():
    """int16[64*64 + 8*24]: attention-policy logit slot -> policy index or -1.
    Slot from*64+to is the plain move; slot 4096 + 24*from_file + 3*to_file + i is
    the promotion to (q, r, b)[i] from rank 7 to rank 8."""
    idx = _move_index()
    out = np.full(64 * 64 + 8 * 24, -1, np.int16)
    for a in range(64):
        for b in range(64):
            if _reachable(a, b):
                out[a * 64 + b] = idx[_name(a) + _name(b)]
    for k in range(8):
        for j in range(8):
            if abs(k - j) <= 1:
                for i, piece in enumerate("qrb"):
                    out[4096 + 24 * k + 3 * j + i] = idx[_name(48 + k) + _name(56 + j) + piece]
    return out


@functools.lru_cache(None)
def conv_policy_map():
    """int16[73*64]: (plane, from-square) of the convolutional policy head ->
    policy index or -1. Planes: 8 directions x 7 distances, 8 knight jumps,
    3 promotion directions x (r, b, q)."""
    idx = _move_index()
    out = np.full(73 * 64, -1, np.int16)
    for sq in range(64):
        x, y = sq % 8, sq // 8
        for d, (dx, dy) in enumerate(_QUEEN_DIRS):
            for dist in range(1, 8):
                tx, ty = x + dx * dist, y + dy * dist
                if 0 <= tx < 8 and 0 <= ty < 8:
                    out[(d * 7 + dist - 1) * 64 + sq] = idx[_name(sq) + _name(ty * 8 + tx)]
        for k, (dx, dy) in enumerate(_KNIGHT):
            tx, ty = x + dx, y + dy
            if 0 <= tx < 8 and 0 <= ty < 8:
                out[(56 + k) * 64 + sq] = idx[_name(sq) + _name(ty * 8 + tx)]
        if y == 6:
            for d, dx in enumerate((-1, 0, 1)):
                tx = x + dx
                if 0 <= tx < 8:
                    for i, piece in enumerate("rbq"):
                        out[(64 + 3 * d + i) * 64 + sq] = idx[_name(sq) + _name(56 + tx) + piece]
    return out


@functools.lru_cache(None)
def pos_encoding():
    """float32[64][64] positional encoding of PE_MAP attention nets: -1 on the
    square itself, 1 on squares a queen or knight reaches from it, else 0."""
    pe = np.zeros((64, 64), np.float32)
    for a in range(64):
        for b in range(64):
            pe[a, b] = -1.0 if a == b else (1.0 if _reachable(a, b) else 0.0)
    return pe
