"""A small CPU interpreter for the PTX the reference emits for streaming kernels, scalar loops and tensor-core tiles.
TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

It executes a `.visible .entry` of the reference's output (tests/golden/*.ref.ptx, produced by
tests/golden/make_reference_ptx.py from the reference's own compiler) for every thread of the launch
at once, with numpy arrays as registers. This is how golden vectors "from the reference itself" exist
without a GPU: integer kernels are reproduced exactly; for float kernels the three hardware
approximations (`sin.approx`, `cos.approx`, `ex2.approx`, whose low bits PTX leaves unspecified) are
evaluated correctly rounded, and `fma.rn.f32` goes through float64 (exact product, one extra rounding of
the sum in rare ties), so float outputs carry the reference's algorithm, not a particular GPU's bits.

Supported: the instructions of `emmyptx/ops.py` and `emmyptx/kernel.py` for one-axis tiles with scalar
global loads and stores, predication, and the early-exit branch to `$L_exit`; and the fully unrolled tensor-core
kernels of `emmyptx/mma.py` (fragments read from global memory as packed 16-bit pairs, `mma.sync.m16n8k16` on
f16 / bf16 with f32 accumulators, converted `.v2.b16` stores, f32 stores and the `red.global.add.f32` of split-K). `mma.sync` is evaluated per warp from the PTX
ISA's fragment lane map (restated in emmyptx/mma.py:6-10) with exact products summed in float64 and rounded to
f32 once per instruction: the hardware's summation order inside one instruction is unspecified, so outputs carry
the reference's algorithm, not one GPU's low bits. Run-time loops (emmyptx/loops.py:231-264) are followed when every
active thread takes the same way at each branch, which holds for loops with static trip counts. Anything else raises.
"""
from __future__ import annotations

import re

import numpy as np

_BUF_SHIFT = 40


class PtxError(NotImplementedError):
    pass


def _f32_literal(tok: str) -> np.float32:
    return np.array([int(tok[2:], 16)], dtype=np.uint32).view(np.float32)[0]


def _bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (h.astype(np.uint32) << np.uint32(16)).view(np.float32)


def _f32_to_bf16(f: np.ndarray) -> np.ndarray:
    """Round to nearest even on the upper 16 bits (tools/run_local.py:31-37 spells the same formula); NaN stays NaN."""
    u = np.ascontiguousarray(f, dtype=np.float32).view(np.uint32)
    r = ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
    return np.where(np.isnan(f), np.uint16(0x7FC0), r)


def _halves_to_f32(h: np.ndarray, kind: str) -> np.ndarray:
    return _bf16_to_f32(h) if kind == "bf16" else h.view(np.float16).astype(np.float32)


class Interpreter:
    def __init__(self, ptx: str) -> None:
        m = re.search(r"\.visible \.entry (\w+)\((.*?)\)\s*(?:\.maxntid[^\n]*\n)?\{(.*)\}", ptx, re.S)
        if m is None:
            raise PtxError("no .visible .entry found")
        self.entry = m.group(1)
        self.params = re.findall(r"\.param \.(\w+) (\w+)", m.group(2))
        self.lines = []
        for raw in m.group(3).splitlines():
            line = raw.split("//")[0].strip()
            if line and not line.startswith(".reg"):
                self.lines.append(line.rstrip(";"))

    def run(self, args: dict, grid: int, block: int) -> None:
        """Execute for grid*block threads. `args`: parameter name -> numpy array (modified in place for outputs)."""
        n = grid * block
        tid = np.arange(n, dtype=np.int64)
        self.special = {"%tid.x": (tid % block).astype(np.int32), "%ctaid.x": (tid // block).astype(np.int32),
                        "%ntid.x": np.full(n, block, np.int32), "%nctaid.x": np.full(n, grid, np.int32)}
        self.bufs = [args[name] for _, name in self.params]
        self.param_addr = {name: np.full(n, (i + 1) << _BUF_SHIFT, np.int64) for i, (_, name) in enumerate(self.params)}
        self.reg: dict = {}
        self.active = np.ones(n, dtype=bool)
        self.n = n
        labels = {line[:-1]: i for i, line in enumerate(self.lines) if line.endswith(":")}
        self.labels, self.parked = labels, {}
        self.jump = None
        pc, executed = 0, 0
        while pc < len(self.lines):
            line = self.lines[pc]
            self.pc = pc
            pc += 1
            if line.endswith(":"):
                waiting = self.parked.pop(line[:-1], None)           # threads that branched forward to this label rejoin
                if waiting is not None:
                    self.active = self.active | waiting
                continue
            self._exec(line)
            executed += 1
            if executed > 50_000_000:
                raise PtxError("instruction budget exhausted (a loop that does not end?)")
            if self.jump is not None:                    # a branch every active thread took (run-time loops)
                if self.jump not in labels:
                    raise PtxError(f"branch to unknown label {self.jump}")
                pc, self.jump = labels[self.jump], None

    # ---- operands -----------------------------------------------------------------------------------
    def _val(self, tok: str, ty: str):
        tok = tok.strip()
        if tok in self.special:
            return self.special[tok]
        if tok.startswith("%"):
            v = self.reg[tok]
            return self._as(v, ty)
        if tok.startswith("0f"):
            return np.full(self.n, _f32_literal(tok), np.float32)
        val = int(tok, 0)
        if ty == "f32":
            raise PtxError(f"integer immediate {tok} in a float slot")
        dt = {"s32": np.int32, "u32": np.uint32, "b32": np.int32, "s64": np.int64, "u64": np.int64, "b64": np.int64,
              "b16": np.uint16}[ty]
        return np.full(self.n, np.array(val).astype(np.int64).astype(dt), dt)

    @staticmethod
    def _as(v, ty: str):
        """Reinterpret a 32-bit register for an instruction type."""
        if ty == "f32":
            return v.view(np.float32) if v.dtype != np.float32 else v
        if ty in ("s32", "b32"):
            return v.view(np.int32) if v.dtype != np.int32 else v
        if ty == "u32":
            return v.view(np.uint32) if v.dtype != np.uint32 else v
        if ty == "pred":
            return v
        return v          # 64-bit values are kept as int64

    def _set(self, dst: str, value, mask=None) -> None:
        value = np.ascontiguousarray(value)
        if value.dtype == np.uint32:
            value = value.view(np.int32)
        m = self.active if mask is None else (self.active & mask)
        if dst in self.reg and not m.all():
            old = self.reg[dst]
            if old.dtype != value.dtype:
                old = old.view(value.dtype)
            value = np.where(m, value, old)
        self.reg[dst] = value

    def _mem(self, tok: str):
        m = re.fullmatch(r"\[(%\w+)(?:\+(-?\d+))?\]", tok.strip())
        if m is None:
            raise PtxError(f"memory operand {tok!r}")
        addr = self.reg[m.group(1)] + int(m.group(2) or 0)
        return (addr >> _BUF_SHIFT) - 1, addr & ((1 << _BUF_SHIFT) - 1)

    # ---- one instruction ------------------------------------------------------------------------------
    def _exec(self, line: str) -> None:
        mask = None
        if line.startswith("@"):
            pred, line = line.split(None, 1)
            neg = pred.startswith("@!")
            p = self.reg[pred[2:] if neg else pred[1:]]
            mask = ~p if neg else p
        op, _, rest = line.partition(" ")
        ops = [t.strip() for t in re.split(r",(?![^\[\{]*[\]\}])", rest)] if rest else []
        parts = op.split(".")
        name = parts[0]
        with np.errstate(all="ignore"):
            self._dispatch(name, parts, ops, mask)

    def _dispatch(self, name, parts, ops, mask) -> None:
        ty = parts[-1]
        V = self._val
        if name == "ret":
            return
        if name == "trap":                                       # the reference's range check of an i64 value (kernel.py:691)
            hit = self.active if mask is None else (self.active & mask)
            if hit.any():
                raise PtxError("the kernel trapped (a 64-bit value does not fit 32 bits)")
            return
        if name == "bra":
            taken = np.ones(self.n, bool) if mask is None else mask
            if ops[0] == "$L_exit":
                self.active = self.active & ~taken
                return
            # A forward branch on which threads diverge (the if / else of a Cond, emmyptx/kernel.py:825-840): the threads
            # that take it wait at the label, the others go on; everybody between here and the label runs masked.
            t = taken[self.active]
            forward = self.labels.get(ops[0], -1) > self.pc
            if forward and (self.parked or (t.any() and not t.all())):
                go = taken & self.active
                self.parked[ops[0]] = self.parked.get(ops[0], np.zeros(self.n, bool)) | go
                self.active = self.active & ~go
                return
            # Any other branch belongs to a run-time loop (emmyptx/loops.py:231-264): its trip count does not depend on
            # the thread, so either every active thread takes it or none does. Divergence is refused.
            if t.size and t.all():
                self.jump = ops[0]
            elif t.any():
                raise PtxError("a backward branch on which the active threads diverge is not supported")
            return
        if name == "activemask":                                  # whole warps run (the launch is a whole number of warps)
            self._set(ops[0], np.full(self.n, -1, np.int32), mask)
            return
        if name == "shfl":
            # shfl.sync.bfly.b32 d, a, delta, clamp, membermask: lane l reads lane l ^ delta of its warp. Threads are laid
            # out block after block and blocks are whole warps, so warp-mates are 32 consecutive positions.
            if parts[2] != "bfly":
                raise PtxError(f"shfl mode {parts[2]!r} is not supported")
            if self.n % 32:
                raise PtxError("shuffles need a whole number of warps")
            delta = int(ops[2], 0)
            src = self.reg[ops[1]]
            partner = np.arange(self.n) ^ delta
            got = src[partner]
            got = np.where(self.active[partner], got, src)           # an inactive source lane returns the caller's own value
            self._set(ops[0], got, mask)
            return
        if name == "ld" and parts[1] == "param":
            self._set(ops[0], self.param_addr[ops[1].strip("[]")])
        elif name == "cvta":
            self._set(ops[0], self.reg[ops[1]])
        elif name == "mov" and ops[1].startswith("{"):            # mov.b32 %b, {%h_lo, %h_hi}
            lo, hi = (self.reg[t.strip()].astype(np.uint32) for t in ops[1].strip("{}").split(","))
            self._set(ops[0], (lo | (hi << np.uint32(16))).astype(np.uint32), mask)
        elif name == "mov":
            src = ops[1]
            if src in self.special:
                self._set(ops[0], self.special[src], mask)
            elif src.startswith("%"):
                self._set(ops[0], self.reg[src], mask)
            elif src.startswith("0f"):
                self._set(ops[0], V(src, "f32"), mask)
            else:
                self._set(ops[0], V(src, "s32" if ty in ("b32", "u32", "s32") else ty), mask)
        elif name == "mma":
            self._mma(parts, ops, mask)
        elif name in ("and", "or", "xor") and ty == "pred":     # and.pred %p, %p1, %p2: predicates are boolean arrays here
            a, b = self.reg[ops[1]].astype(bool), self.reg[ops[2]].astype(bool)
            self._set(ops[0], {"and": np.logical_and, "or": np.logical_or, "xor": np.logical_xor}[name](a, b), mask)
        elif name in ("and", "or", "xor"):
            a, b = V(ops[1], "s32"), V(ops[2], "s32")
            self._set(ops[0], {"and": np.bitwise_and, "or": np.bitwise_or, "xor": np.bitwise_xor}[name](a, b), mask)
        elif name == "shr":
            a, b = V(ops[1], ty), V(ops[2], "u32").astype(np.int64)
            self._set(ops[0], (a.astype(np.int64) >> np.minimum(b, 31)).astype(a.dtype) if ty == "s32" else
                      (a.astype(np.uint32) >> np.minimum(b, 31).astype(np.uint32)), mask)
        elif name == "shl":
            a, b = V(ops[1], "u32"), V(ops[2], "u32")
            self._set(ops[0], (a.astype(np.uint64) << b.astype(np.uint64)).astype(np.uint32), mask)
        elif name in ("add", "sub", "mul", "mad", "div", "rem", "max", "min", "abs", "neg") and ty in ("s32", "u32", "s64", "u64"):
            self._int_arith(name, parts, ops, mask)
        elif name in ("add", "sub", "mul", "div", "max", "min") and ty == "f32":
            a, b = V(ops[1], "f32"), V(ops[2], "f32")
            f = {"add": np.add, "sub": np.subtract, "mul": np.multiply, "div": np.divide, "max": np.fmax, "min": np.fmin}[name]
            self._set(ops[0], f(a, b).astype(np.float32), mask)
        elif name == "fma":
            a, b, c = (V(t, "f32").astype(np.float64) for t in ops[1:4])
            self._set(ops[0], (a * b + c).astype(np.float32), mask)
        elif name in ("abs", "neg") and ty == "f32":
            a = V(ops[1], "f32")
            self._set(ops[0], np.abs(a) if name == "abs" else -a, mask)
        elif name == "copysign":                                  # sign of the first source, magnitude of the second
            self._set(ops[0], np.copysign(V(ops[2], "f32"), V(ops[1], "f32")), mask)
        elif name in ("rcp", "sqrt"):
            a = V(ops[1], "f32")
            self._set(ops[0], (np.float32(1) / a if name == "rcp" else np.sqrt(a)).astype(np.float32), mask)
        elif name in ("sin", "cos", "ex2", "lg2"):
            a = V(ops[1], "f32").astype(np.float64)
            f = {"sin": np.sin, "cos": np.cos, "ex2": np.exp2, "lg2": np.log2}[name]
            self._set(ops[0], f(a).astype(np.float32), mask)
        elif name == "cvt":
            self._cvt(parts, ops, mask)
        elif name == "setp":
            cmp, cty = parts[1], parts[2]
            a, b = V(ops[1], cty), V(ops[2], cty)
            if cmp == "nan":
                r = np.isnan(a) | np.isnan(b)
            else:
                unordered = cmp.endswith("u") and cmp not in ("lu",) and cty == "f32" and cmp in ("neu", "equ", "ltu", "leu", "gtu", "geu")
                base = cmp[:-1] if unordered else cmp
                r = {"eq": np.equal, "ne": np.not_equal, "lt": np.less, "le": np.less_equal, "gt": np.greater,
                     "ge": np.greater_equal}[base](a, b)
                if unordered:
                    r = r | np.isnan(a) | np.isnan(b)
            self._set(ops[0], r, mask)
        elif name == "selp":
            a, b = V(ops[1], ty), V(ops[2], ty)
            self._set(ops[0], np.where(self.reg[ops[3]], a, b), mask)
        elif name == "ld" and parts[1] == "global":
            buf, off = self._mem(ops[1])
            dt = np.float32 if ty == "f32" else (np.uint16 if ty == "b16" else (np.int64 if ty in ("s64", "u64", "b64") else np.int32))
            dsts = [t.strip() for t in ops[0].strip("{}").split(",")]        # one register, or the members of a .v2 / .v4
            m = self.active if mask is None else self.active & mask
            for j, dst in enumerate(dsts):                                   # (two adjacent f32 loads pair up: emmyptx/kernel.py:517-548)
                out = np.zeros(self.n, dt)
                for b in np.unique(buf[m]):
                    sel = m & (buf == b)
                    arr = self.bufs[int(b)].reshape(-1)
                    out[sel] = arr.view(dt)[off[sel] // out.itemsize + j]
                self._set(dst, out, mask)
        elif name == "st" and parts[1] == "global":
            buf, off = self._mem(ops[0])
            width = 2 if ty == "b16" else 4
            srcs = [t.strip() for t in ops[1].strip("{}").split(",")]        # one value, or the members of a .v2
            m = self.active if mask is None else self.active & mask
            for j, tok in enumerate(srcs):
                val = self.reg[tok] if ty == "b16" else V(tok, ty)
                for b in np.unique(buf[m]):
                    sel = m & (buf == b)
                    arr = self.bufs[int(b)].reshape(-1)
                    arr.view(val.dtype)[(off[sel] + j * width) // width] = val[sel]
        elif name == "red" and tuple(parts[1:]) == ("global", "add", "f32"):
            # split-K partial sums (emmyptx/mma.py:239-240). The hardware adds them in no particular order; here in thread order.
            buf, off = self._mem(ops[0])
            val = V(ops[1], "f32")
            m = self.active if mask is None else self.active & mask
            for b in np.unique(buf[m]):
                sel = m & (buf == b)
                arr = self.bufs[int(b)].reshape(-1).view(np.float32)
                np.add.at(arr, off[sel] // 4, val[sel])
        else:
            raise PtxError(f"unsupported instruction {'.'.join(parts)}")

    def _mma(self, parts, ops, mask) -> None:
        """mma.sync.aligned.m16n8k16.row.col.f32.<ab>.<ab>.f32 {d}, {a}, {b}, {c}: every warp multiplies its 16x16 A by
        its 16x8 B. Lane (g, t) = (lane / 4, lane % 4) holds a[i] = A[g + 8 (i & 1)][2t + 8 (i >> 1) + {0, 1}],
        b[i] = B[2t + 8 i + {0, 1}][g], c[i] = C[g + 8 (i >> 1)][2t + (i & 1)], low half of a pair first."""
        if mask is not None or not self.active.reshape(-1, 32).all(axis=1).any() or self.n % 32:
            raise PtxError("mma.sync needs whole warps")
        if tuple(parts[1:6]) != ("sync", "aligned", "m16n8k16", "row", "col") or parts[6] != "f32" or parts[9] != "f32":
            raise PtxError(f"unsupported {'.'.join(parts)}")
        kind = parts[7]
        groups = [[t.strip() for t in o.strip("{}").split(",")] for o in ops]
        d_regs, a_regs, b_regs, c_regs = groups
        w = self.n // 32
        lanes = np.arange(32)
        g, t = lanes // 4, lanes % 4
        A = np.zeros((w, 16, 16), np.float64)
        B = np.zeros((w, 16, 8), np.float64)
        C = np.zeros((w, 16, 8), np.float64)
        for i, r in enumerate(a_regs):
            u = self.reg[r].view(np.uint32).reshape(w, 32)
            for j in (0, 1):
                h = ((u >> np.uint32(16 * j)) & np.uint32(0xFFFF)).astype(np.uint16)
                A[:, g + 8 * (i & 1), 2 * t + 8 * (i >> 1) + j] = _halves_to_f32(h, kind)
        for i, r in enumerate(b_regs):
            u = self.reg[r].view(np.uint32).reshape(w, 32)
            for j in (0, 1):
                h = ((u >> np.uint32(16 * j)) & np.uint32(0xFFFF)).astype(np.uint16)
                B[:, 2 * t + 8 * i + j, g] = _halves_to_f32(h, kind)
        for i, r in enumerate(c_regs):
            C[:, g + 8 * (i >> 1), 2 * t + (i & 1)] = self._as(self.reg[r], "f32").reshape(w, 32)
        D = (A @ B + C).astype(np.float32)
        for i, r in enumerate(d_regs):
            self._set(r, np.ascontiguousarray(D[:, g + 8 * (i >> 1), 2 * t + (i & 1)]).reshape(-1))

    def _int_arith(self, name, parts, ops, mask) -> None:
        V = self._val
        ty = parts[-1]
        if name == "mul" and parts[1] == "wide":
            a, b = V(ops[1], ty).astype(np.int64), V(ops[2], ty).astype(np.int64)
            self._set(ops[0], a * b, mask)
            return
        if ty in ("s64", "u64"):
            a, b = self.reg[ops[1]] if ops[1].startswith("%") else V(ops[1], "s64"), \
                   self.reg[ops[2]] if ops[2].startswith("%") else V(ops[2], "s64")
            self._set(ops[0], {"add": np.add, "sub": np.subtract}[name](a, b), mask)
            return
        wide = [V(t, ty).astype(np.int64) for t in ops[1:]]
        if name == "mad":
            r = wide[0] * wide[1] + wide[2]
        elif name in ("add", "sub", "mul"):
            r = {"add": np.add, "sub": np.subtract, "mul": np.multiply}[name](wide[0], wide[1])
        elif name in ("div", "rem"):
            a, b = wide
            q = np.abs(a) // np.where(b == 0, 1, np.abs(b))
            q = np.where((a < 0) != (b < 0), -q, q)                # truncates toward zero, as div.s32
            r = q if name == "div" else a - q * b
        elif name in ("max", "min"):
            r = (np.maximum if name == "max" else np.minimum)(wide[0], wide[1])
        elif name == "abs":
            r = np.abs(wide[0])
        else:
            r = -wide[0]
        dt = np.uint32 if ty == "u32" else np.int32
        self._set(ops[0], (r & 0xFFFFFFFF).astype(np.uint32).view(np.int32) if dt == np.int32 else (r & 0xFFFFFFFF).astype(np.uint32), mask)

    def _cvt(self, parts, ops, mask) -> None:
        V = self._val
        mods = parts[1:]
        dst_ty, src_ty = mods[-2], mods[-1]
        rnd = mods[0] if len(mods) == 3 else None
        if dst_ty == "f32" and src_ty in ("f16", "bf16"):       # widening a 16-bit element (exact)
            h = np.asarray(self.reg[ops[1]]).astype(np.uint16)
            wide = h.view(np.float16).astype(np.float32) if src_ty == "f16" else (h.astype(np.uint32) << np.uint32(16)).view(np.float32)
            self._set(ops[0], wide, mask)
            return
        a = V(ops[1], src_ty)
        if dst_ty == "f32" and src_ty == "f32":
            f = {"rni": np.rint, "rzi": np.trunc, "rmi": np.floor, "rpi": np.ceil}[rnd]
            self._set(ops[0], f(a).astype(np.float32), mask)
        elif dst_ty == "s32" and src_ty == "f32":
            f = {"rni": np.rint, "rzi": np.trunc, "rmi": np.floor, "rpi": np.ceil}[rnd]
            v = np.nan_to_num(f(a.astype(np.float64)), nan=0.0)
            self._set(ops[0], np.clip(v, -2**31, 2**31 - 1).astype(np.int32), mask)
        elif dst_ty == "f32" and src_ty in ("s32", "u32"):
            self._set(ops[0], a.astype(np.float32), mask)
        elif dst_ty in ("f16", "bf16") and src_ty == "f32" and rnd == "rn":
            h = _f32_to_bf16(a) if dst_ty == "bf16" else a.astype(np.float16).view(np.uint16)
            self._set(ops[0], h, mask)
        elif dst_ty == "s32" and src_ty == "s64":               # i64 buffers carry 32-bit values (emmyptx/kernel.py:41, 685-691)
            self._set(ops[0], np.asarray(a, np.int64).astype(np.int32), mask)
        elif dst_ty == "s64" and src_ty == "s32":
            self._set(ops[0], np.asarray(a, np.int32).astype(np.int64), mask)
        else:
            raise PtxError(f"unsupported conversion {'.'.join(parts)}")


def run_entry(ptx: str, args: dict, grid: int, block: int) -> None:
    Interpreter(ptx).run(args, grid, block)
