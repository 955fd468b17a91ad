"""TOSA-text front end: reads the single-function TOSA 1.0 MLIR modules the reference keeps
as op fixtures (tests/testdata/tosa_ops/*.mlir, tests/testdata/gen_ops/*.mlir: what
tosa-converter-for-tflite emits) and builds the equivalent op-list Graph, fusing the chains
the reference's Linalg->TorqHL patterns fuse:

    conv2d / depthwise_conv2d -> rescale [-> clamp]                       one conv record
    rescale(i8->i32), rescale(i8->i32) -> add|sub|mul -> rescale(i32->i8) one add/sub/mul record
    pad(const) -> max_pool2d                                              max pool with pad value
    rescale(i8->i8), table, avg_pool2d, max_pool2d, reshape, resize(2x nearest), concat

(compiler/torq/Conversions/LinalgToTorqHL/Conv2DPattern.cpp:587-647,
ElementWiseBinaryPattern.cpp:439-456, PoolingPattern.cpp:160, ClampPattern.cpp:349-454.)
Anything else raises NotImplementedError with the op name. It is a reader for the textual
form only (the generic MLIR parser lives in the absent IREE/LLVM tree).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field

import numpy as np

from .oplist import Graph, TensorRef

_NP = {"i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64, "index": np.int64, "f32": np.float32}


@dataclass
class _Val:
    name: str
    shape: tuple
    dtype: str
    const: np.ndarray | None = None
    op: "_Op | None" = None


@dataclass
class _Op:
    name: str
    operands: list
    attrs: dict
    result: _Val | None = None
    users: list = field(default_factory=list)


def _parse_type(t: str):
    t = t.strip()
    m = re.match(r"tensor<(.*)>", t)
    if not m:
        m2 = re.match(r"!tosa\.shape<(\d+)>", t)
        if m2:
            return (int(m2.group(1)),), "index"
        raise ValueError(f"unsupported type {t}")
    mm = re.match(r"^((?:\d+x)*)(\w+)$", m.group(1))
    if not mm:
        raise NotImplementedError(f"unsupported tensor type {t}")
    return tuple(int(p) for p in mm.group(1).split("x") if p), mm.group(2)


def _parse_dense(body: str, shape, dtype):
    np_t = _NP[dtype]
    body = body.strip()
    n = int(np.prod(shape)) if shape else 1
    if body.startswith('"0x'):
        raw = bytes.fromhex(body[3:-1])
        return np.frombuffer(raw, dtype=np_t)[:n].reshape(shape).copy()
    if body.startswith("["):
        vals = [int(v) if dtype != "f32" else float(v) for v in re.findall(r"-?\d+(?:\.\d+)?(?:[eE][-+]?\d+)?", body)]
        return np.array(vals, dtype=np_t).reshape(shape)
    v = {"true": 1, "false": 0}.get(body, None)
    if v is None:
        v = float(body) if dtype == "f32" else int(body)
    return np.full(shape, v, dtype=np_t)


def _parse_attrs(text: str) -> dict:
    out = {}
    for k, v in re.findall(r"(\w+)\s*=\s*(array<i64:[^>]*>|\"[^\"]*\"|[-\w\.]+(?:\s*:\s*\w+)?)", text):
        if v.startswith("array<"):
            out[k] = [int(x) for x in re.findall(r"-?\d+", v.split(":", 1)[1])]
        elif v.startswith('"'):
            out[k] = v.strip('"')
        else:
            tok = v.split(":")[0].strip()
            out[k] = {"true": True, "false": False}.get(tok, None)
            if out[k] is None:
                try:
                    out[k] = int(tok)
                except ValueError:
                    out[k] = tok
    return out


def parse_module(text: str):
    """Returns (inputs [_Val], ops [_Op], returned [_Val])."""
    text = re.sub(r"//[^\n]*", "", text)
    vals: dict[str, _Val] = {}
    ops: list[_Op] = []
    m = re.search(r"func\.func\s+@\w+\((.*?)\)\s*->", text, re.S)
    if not m:
        raise ValueError("no func.func found")
    inputs = []
    for name, ty in re.findall(r"(%\w+)\s*:\s*(tensor<[^>]*>)", m.group(1)):
        shape, dt = _parse_type(ty)
        vals[name] = _Val(name, shape, dt)
        inputs.append(vals[name])
    body = text[m.end():]
    body = body[body.index("\n") + 1:] if "\n" in body else ""  # rest of the signature line: result types, attributes
    returned = []
    for line in body.split("\n"):
        line = line.strip()
        if not line or line in ("}", "{"):
            continue
        r = re.match(r"return\s+(.*?)\s*:", line)
        if r:
            returned = [vals[n.strip()] for n in r.group(1).split(",")]
            continue
        c = re.match(r"(%\w+)\s*=\s*(?:\"tosa\.const\"\(\)\s*<\{values\s*=\s*|arith\.constant\s+|tosa\.const_shape\s*\{values\s*=\s*)"
                     r"dense<(.*)>\s*:\s*(tensor<[^>]*>)", line)
        if c:
            shape, dt = _parse_type(c.group(3))
            vals[c.group(1)] = _Val(c.group(1), shape, dt, const=_parse_dense(c.group(2), shape, dt))
            continue
        o = re.match(r"(%\w+)\s*=\s*\"?tosa\.(\w+)\"?\s*\(?([^{:]*?)\)?\s*(?:<?\{(.*?)\}>?)?\s*:\s*\(.*\)\s*->\s*(.*)$", line)
        if o:
            res_name, opname, operand_text, attr_text, res_type = o.groups()
            operands = [vals[n] for n in re.findall(r"%\w+", operand_text)]
            shape, dt = _parse_type(res_type)
            op = _Op(opname, operands, _parse_attrs(attr_text or ""))
            op.result = _Val(res_name, shape, dt, op=op)
            vals[res_name] = op.result
            for v in operands:
                if v.op is not None:
                    v.op.users.append(op)
            ops.append(op)
            continue
        if line.startswith("module") or line.startswith("func.func") or line.startswith("{-#") or line.startswith("#"):
            continue
        raise NotImplementedError(f"cannot read line: {line[:120]}")
    return inputs, ops, returned


def _scalar(v: _Val) -> int:
    if v.const is None:
        raise NotImplementedError("expected a constant operand")
    return int(v.const.reshape(-1)[0])


def build_graph(text: str) -> Graph:
    inputs, ops, returned = parse_module(text)
    g = Graph()
    env: dict[str, TensorRef] = {}
    for v in inputs:
        env[v.name] = g.input(v.shape, v.dtype)
    done: set[int] = set()

    def rescale_params(op):
        x, mult, shift, izp, ozp = op.operands
        return dict(x=x, mult=mult.const.reshape(-1).astype(np.int32), shift=shift.const.reshape(-1).astype(np.int8),
                    izp=_scalar(izp), ozp=_scalar(ozp), per_channel=bool(op.attrs.get("per_channel", False)),
                    double_round="DOUBLE" in str(op.attrs.get("rounding_mode", "SINGLE_ROUND")))

    def only_user(op, name):
        users = list({id(u): u for u in op.users}.values())
        return users[0] if len(users) == 1 and users[0].name == name else None

    def fold_clamp(op, lo=-128, hi=127):
        """Follow an optional tosa.clamp after `op`; returns (last op of the chain, lo, hi)."""
        c = only_user(op, "clamp")
        if c is not None:
            done.add(id(c))
            return c, max(lo, int(c.attrs["min_val"])), min(hi, int(c.attrs["max_val"]))
        return op, lo, hi

    for op in ops:
        if id(op) in done:
            continue
        n = op.name
        if n in ("conv2d", "depthwise_conv2d"):
            x, w, bias, izp, wzp = op.operands
            rs = only_user(op, "rescale")
            if rs is None or w.const is None:
                raise NotImplementedError(f"{n} without a constant weight and a following rescale")
            done.add(id(rs))
            p = rescale_params(rs)
            last, lo, hi = fold_clamp(rs)
            fn = g.conv2d if n == "conv2d" else g.depthwise_conv2d
            mult, shift = (p["mult"], p["shift"]) if p["per_channel"] else (p["mult"][:1], p["shift"][:1])
            y = fn(env[x.name], w.const, bias.const.reshape(-1), mult, shift, stride=tuple(op.attrs["stride"]),
                   dilation=tuple(op.attrs["dilation"]), pad=tuple(op.attrs["pad"]), input_zp=_scalar(izp),
                   weight_zp=_scalar(wzp), out_zp=p["ozp"], clamp=(lo, hi), double_round=p["double_round"])
            env[last.result.name] = y
        elif n == "rescale":
            p = rescale_params(op)
            src = op.operands[0]
            if src.dtype == "i8" and op.result.dtype == "i32":
                users = list({id(u): u for u in op.users}.values())  # x + x uses the rescale twice
                if len(users) == 1 and users[0].name == "rescale" and users[0].result.dtype == "i32":
                    users = list({id(u): u for u in users[0].users}.values())  # first of two input stages
                if len(users) != 1 or users[0].name not in ("add", "sub", "mul"):
                    raise NotImplementedError("i8->i32 rescale that does not feed add/sub/mul")
                continue  # consumed when the binary op is reached
            if src.dtype == "i32" and op.result.dtype == "i32" and src.op is not None and src.op.name == "rescale" and \
                    src.op.operands[0].dtype == "i8":
                users = list({id(u): u for u in op.users}.values())
                if len(users) != 1 or users[0].name not in ("add", "sub", "mul"):
                    raise NotImplementedError("i32->i32 rescale that does not feed add/sub/mul")
                continue  # second input stage, consumed when the binary op is reached
            if src.dtype == "i8" and op.result.dtype == "i8":
                last, lo, hi = fold_clamp(op)
                mult, shift = (p["mult"], p["shift"]) if p["per_channel"] else (p["mult"][:1], p["shift"][:1])
                env[last.result.name] = g.rescale(env[src.name], mult, shift, input_zp=p["izp"], out_zp=p["ozp"],
                                                  clamp=(lo, hi), double_round=p["double_round"])
            else:
                raise NotImplementedError(f"rescale {src.dtype}->{op.result.dtype} outside a fused chain")
        elif n in ("add", "sub", "mul"):
            a, b = op.operands[0], op.operands[1]
            if a.op is None or b.op is None or a.op.name != "rescale" or b.op.name != "rescale":
                raise NotImplementedError(f"{n} whose operands are not i8->i32 rescales")
            rs = only_user(op, "rescale")
            if rs is None:
                raise NotImplementedError(f"{n} without an output rescale")
            done.add(id(rs))
            po = rescale_params(rs)
            if po["izp"] != 0:
                raise NotImplementedError("output rescale of a binary op with a non-zero input zero point")

            def input_side(v):
                """(source i8 value, zero point, left shift, multiplier, shift) of one operand. Two forms:
                one rescale i8->i32, or the TFLite-derived pair: i8->i32 with multiplier 2^30 and shift
                s <= 30 (an exact left shift by 30 - s), then i32->i32 with the real multiplier."""
                p2 = rescale_params(v.op)
                if p2["ozp"] != 0 or p2["per_channel"] or p2["double_round"] != po["double_round"]:
                    raise NotImplementedError("input rescale with an output zero point, per channel, or another rounding mode")
                src = p2["x"]
                if src.dtype == "i8":
                    return src, p2["izp"], 0, int(p2["mult"][0]), int(p2["shift"][0])
                if src.dtype == "i32" and src.op is not None and src.op.name == "rescale" and src.op.operands[0].dtype == "i8":
                    p1 = rescale_params(src.op)
                    s1 = int(p1["shift"][0])
                    if int(p1["mult"][0]) != 1 << 30 or not 8 <= s1 <= 30 or p1["ozp"] != 0 or p2["izp"] != 0 or p1["per_channel"]:
                        raise NotImplementedError("first input stage that is not an exact left shift")
                    return p1["x"], p1["izp"], 30 - s1, int(p2["mult"][0]), int(p2["shift"][0])
                raise NotImplementedError(f"{n} whose operands are not i8->i32 rescales")

            xa, za, la, ma, sa = input_side(a)
            xb, zb, lb, mb, sb = input_side(b)
            last, lo, hi = fold_clamp(rs)
            fn = getattr(g, n)
            env[last.result.name] = fn(env[xa.name], env[xb.name], a_zp=za, a_ms=(ma, sa), b_zp=zb, b_ms=(mb, sb),
                                       out_ms=(int(po["mult"][0]), int(po["shift"][0])), out_zp=po["ozp"], clamp=(lo, hi),
                                       double_round=po["double_round"], a_lshift=la, b_lshift=lb)
        elif n == "table":
            env[op.result.name] = g.table(env[op.operands[0].name], op.operands[1].const.reshape(-1))
        elif n == "pad":
            mp = only_user(op, "max_pool2d")
            if mp is None:
                raise NotImplementedError("tosa.pad that does not feed max_pool2d")
            continue
        elif n == "max_pool2d":
            src = op.operands[0]
            pad = list(op.attrs["pad"])
            pad_value = -32768 if src.dtype == "i16" else -128  # the type's lowest value: padding never wins
            if src.op is not None and src.op.name == "pad":
                amounts = src.op.operands[1].const.reshape(-1)  # [n0,n1,h0,h1,w0,w1,c0,c1]
                pad = [pad[0] + int(amounts[2]), pad[1] + int(amounts[3]), pad[2] + int(amounts[4]), pad[3] + int(amounts[5])]
                pad_value = _scalar(src.op.operands[2])
                src = src.op.operands[0]
            env[op.result.name] = g.maxpool2d(env[src.name], tuple(op.attrs["kernel"]), tuple(op.attrs["stride"]),
                                              tuple(pad), pad_value)
        elif n == "avg_pool2d":
            x, izp, ozp = op.operands
            env[op.result.name] = g.avg_pool2d(env[x.name], tuple(op.attrs["kernel"]), tuple(op.attrs["stride"]),
                                               tuple(op.attrs["pad"]), _scalar(izp), _scalar(ozp))
        elif n == "reshape":
            env[op.result.name] = g.reshape(env[op.operands[0].name], op.result.shape)
        elif n == "resize":
            x = op.operands[0]
            if op.attrs.get("mode") != "NEAREST_NEIGHBOR" or op.result.shape[1] != 2 * x.shape[1] or op.result.shape[2] != 2 * x.shape[2]:
                raise NotImplementedError("only 2x nearest-neighbour resize")
            env[op.result.name] = g.resize_nearest_2x(env[x.name])
        elif n == "concat":
            a, b = op.operands
            if int(op.attrs.get("axis", -1)) != len(a.shape) - 1:
                raise NotImplementedError("concat along a non-channel axis")
            one = (1 << 30, 30)
            env[op.result.name] = g.concat(env[a.name], env[b.name], a_zp=0, a_ms=one, b_zp=0, b_ms=one, out_zp=0)
        elif n == "matmul":
            a, b, azp, bzp = op.operands
            if a.dtype != "i8" or b.dtype != "i8" or op.result.dtype != "i32" or len(a.shape) != 3 or a.shape[0] != 1:
                raise NotImplementedError("tosa.matmul other than one batch of i8 x i8 -> i32")
            y = g.matmul_i32(g.reshape(env[a.name], a.shape[1:]), g.reshape(env[b.name], b.shape[1:]), a_zp=_scalar(azp),
                             b_zp=_scalar(bzp))
            env[op.result.name] = g.reshape(y, op.result.shape)
        elif n == "clamp":
            x = op.operands[0]
            if x.dtype != "i8":
                raise NotImplementedError("clamp that does not follow a rescale")
            # on its own: the identity rescale (multiplier 2^30, shift 30 is exact) with the clamp range
            env[op.result.name] = g.rescale(env[x.name], np.array([1 << 30], np.int32), np.array([30], np.int8), input_zp=0,
                                            out_zp=0, clamp=(max(-128, int(op.attrs["min_val"])), min(127, int(op.attrs["max_val"]))),
                                            double_round=False)
        elif n == "identity":
            x = op.operands[0]
            env[op.result.name] = g.reshape(env[x.name], x.shape)
        else:
            raise NotImplementedError(f"tosa.{n}")
    for v in returned:
        g.output(env[v.name])
    return g


def build_graph_from_file(path: str) -> Graph:
    with open(path) as f:
        return build_graph(f.read())
