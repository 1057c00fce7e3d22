"""CPU restatement of what each collective must produce: out = fold(op, per-rank inputs).

Floating types fold in float64 and round once; integers wrap in their own
width like the kernels; ``avg`` is the sum divided by the number of ranks
(truncating division for integers). bfloat16 travels as uint16 bit patterns.
"""
import numpy as np

INT_TYPES = (np.int8, np.uint8, np.int32, np.uint32, np.int64, np.uint64)


def bf16_to_f32(u16):
    u16 = np.asarray(u16, dtype=np.uint16)
    return (u16.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(f32):
    u = np.asarray(f32, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    out = rounded.astype(np.uint16)
    nan = np.isnan(np.asarray(f32, dtype=np.float32))
    if np.any(nan):
        out = np.where(nan, np.uint16(0x7FC0), out)
    return out


def fold(inputs, op, bf16=False):
    """inputs: list of equally shaped arrays, one per rank. Returns the reduced array."""
    n = len(inputs)
    if bf16:
        vals = [bf16_to_f32(x).astype(np.float64) for x in inputs]
    elif inputs[0].dtype.type in INT_TYPES:
        dt = inputs[0].dtype
        acc = inputs[0].copy()
        with np.errstate(over="ignore"):
            for x in inputs[1:]:
                if op in ("sum", "avg"):
                    acc = (acc + x).astype(dt)
                elif op == "prod":
                    acc = (acc * x).astype(dt)
                elif op == "max":
                    acc = np.maximum(acc, x)
                elif op == "min":
                    acc = np.minimum(acc, x)
            if op == "avg":
                if np.issubdtype(dt, np.signedinteger):
                    acc = np.trunc(acc.astype(np.float64) / n).astype(dt) if dt.itemsize < 8 else (np.sign(acc) * (np.abs(acc) // n)).astype(dt)
                else:
                    acc = (acc // np.array(n, dtype=dt)).astype(dt)
        return acc
    else:
        vals = [x.astype(np.float64) for x in inputs]
    acc = vals[0].copy()
    for v in vals[1:]:
        if op in ("sum", "avg"):
            acc = acc + v
        elif op == "prod":
            acc = acc * v
        elif op == "max":      # IEEE maxNum / minNum: a NaN loses against a number (the library's rule, and NCCL's)
            acc = np.fmax(acc, v)
        elif op == "min":
            acc = np.fmin(acc, v)
    if op == "avg":
        acc = acc / n
    if bf16:
        return f32_to_bf16(acc.astype(np.float32))
    return acc.astype(inputs[0].dtype)


def ring_fold_sum(inputs, align=1):
    """fp32 / fp64 sum in the order the ring algorithm adds: the vector is cut into world slots of ceil(count / world)
    elements (rounded up to `align` elements: 1 on the host, one 16-byte vector in the device kernels); slot j starts
    at rank j and picks up ranks j+1, j+2, ... one by one. Bit-exact reference for the ring all-reduce
    (floating-point addition is commutative but not associative)."""
    n = len(inputs)
    count = inputs[0].size
    per = -(-count // n)
    per = -(-per // align) * align
    out = np.empty_like(inputs[0])
    for j in range(n):
        lo, hi = min(per * j, count), min(per * (j + 1), count)
        acc = inputs[j][lo:hi].copy()
        for k in range(1, n):
            acc = acc + inputs[(j + k) % n][lo:hi]
        out[lo:hi] = acc
    return out


def tolerances(dtype_name, world):
    """(rtol, atol) the tests use when comparing a kernel with the fold above."""
    return {
        "float32": (1e-5, 1e-6 * world),
        "float64": (1e-12, 1e-13 * world),
        "float16": (4e-3, 4e-3 * world),
        "bfloat16": (2e-2, 2e-2 * world),
    }.get(dtype_name, (0.0, 0.0))


def make_input(dtype_name, count, seed, kind="uniform"):
    """Seeded per-rank input: floats uniform[-1,1] or normal(0,1); integers uniform in [-1000,1000]
    (unsigned: [0,1000]; 8-bit: +-12 so that sums stay in range). bfloat16 comes back as uint16 bits."""
    rng = np.random.default_rng(seed)
    if dtype_name in ("float16", "float32", "float64", "bfloat16"):
        v = rng.uniform(-1.0, 1.0, count) if kind == "uniform" else rng.normal(0.0, 1.0, count)
        if dtype_name == "bfloat16":
            return f32_to_bf16(v.astype(np.float32))
        return v.astype(dtype_name)
    dt = np.dtype(dtype_name)
    span = 12 if dt.itemsize == 1 else 1000
    lo = 0 if np.issubdtype(dt, np.unsignedinteger) else -span
    return rng.integers(lo, span + 1, count).astype(dt)
