"""Writes the golden fixtures under tests/golden/.

mismatch_2x16.actp is assembled here byte by byte with `struct.pack`, straight from the layout the
reference documents (src/tensor/wire/format.zig:1-26, per-op payloads in encode.zig:136-230) and
the operation list `tensor.define` records for the README's `mismatch` program (Builder rules,
src/tensor/trace/builder.zig:322-330,476-485,573-587).  It does not go through this repository's
encoder, so the encoder and both decoders can be checked against it.

mismatch_16_known_answers.json holds the reference's shipped known answers for that program
(README.md:151-153, examples/consumer/src/main.zig:200-228) and the f32 [2,3]x[3,2] dot
(src/executable/fragment.zig:1193-1205).

Run:  python tests/golden/make_golden.py
"""
import json
import os
import struct

HERE = os.path.dirname(os.path.abspath(__file__))

F32 = 11
KIND = {"parameter": 0, "constant": 1, "unary": 2, "binary": 3, "broadcast_in_dim": 6, "reduce": 9}
SIN, MUL, SUB, SUM = 6, 2, 1, 0


def u32(v):
    return struct.pack("<I", v)


def i64(v):
    return struct.pack("<q", v)


def blob(b):
    return u32(len(b)) + b


def dims(ds):
    out = u32(len(ds))
    for name, extent in ds:
        out += blob(name.encode()) + i64(extent)
    return out


def ints(vs):
    return u32(len(vs)) + b"".join(i64(v) for v in vs)


def mismatch_program(guesses, points):
    full = [("guess", guesses), ("point", points)]
    ops = [
        u32(KIND["parameter"]) + u32(F32) + dims([("guess", guesses)]),          # %0 frequency
        u32(KIND["parameter"]) + u32(F32) + dims([("point", points)]),           # %1 time
        u32(KIND["parameter"]) + u32(F32) + dims([("point", points)]),           # %2 sample
        u32(KIND["broadcast_in_dim"]) + dims(full) + u32(0) + ints([0]),          # %3
        u32(KIND["broadcast_in_dim"]) + dims(full) + u32(1) + ints([1]),          # %4
        u32(KIND["binary"]) + u32(MUL) + u32(3) + u32(4),                         # %5 frequency*time
        u32(KIND["unary"]) + u32(SIN) + u32(5),                                   # %6 sin
        u32(KIND["broadcast_in_dim"]) + dims(full) + u32(2) + ints([1]),          # %7
        u32(KIND["binary"]) + u32(SUB) + u32(6) + u32(7),                         # %8 gap
        u32(KIND["binary"]) + u32(MUL) + u32(8) + u32(8),                         # %9 gap*gap
        u32(KIND["constant"]) + u32(F32) + dims([]) + blob(struct.pack("<f", 0.0)),  # %10 init
        u32(KIND["reduce"]) + u32(9) + u32(10) + u32(SUM) + ints([1]),            # %11 sum over point
    ]
    return b"ACTP" + u32(1) + blob(b"mismatch") + u32(len(ops)) + b"".join(ops) + u32(1) + u32(11)


def main():
    with open(os.path.join(HERE, "mismatch_2x16.actp"), "wb") as f:
        f.write(mismatch_program(2, 16))
    answers = {
        "mismatch": {"points": 16, "time_step": 0.25, "true_frequency": 3.0,
                     "frequency": [2.5, 3.0], "value": [8.656, 0.0], "abs_tolerance": [1e-3, 1e-9]},
        "dot_f32_2x3_3x2": {"lhs": [1, 2, 3, 4, 5, 6], "rhs": [7, 8, 9, 10, 11, 12], "out": [58, 64, 139, 154]},
    }
    with open(os.path.join(HERE, "known_answers.json"), "w") as f:
        json.dump(answers, f, indent=1)


if __name__ == "__main__":
    main()
