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

from .oplist import ACTIVATION, Graph, TensorRef

_NP = {"i8": np.int8, "i16": np.int16, "i32": np.int32, "i64": np.int64, "index": np.int64, "f32": np.float32,
       "i1": np.int8, "ui8": np.uint8, "ui16": np.uint16, "bf16": np.uint16, "i48": np.int64}
# element type of the op-list tensor that holds a TOSA value: booleans are 0 / 1 bytes, unsigned types keep their
# bits in the signed type of the same width (tosa.rescale's input_unsigned / output_unsigned say how to read them)
_GRAPH_DTYPE = {"i1": "i8", "ui8": "i8", "ui16": "i16"}


def graph_dtype(dtype: str) -> str:
    return _GRAPH_DTYPE.get(dtype, dtype)


def _to_bf16_bits(values) -> np.ndarray:
    u = np.asarray(values, np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


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
    # a dynamic extent is specialised to 1, as the reference's test harness does when it draws the inputs of such a
    # function (python/torq/testing/iree.py:385): an executable of this backend has static shapes
    mm = re.match(r"^((?:(?:\d+|\?)x)*)(\w+)$", m.group(1))
    if not mm:
        raise NotImplementedError(f"unsupported tensor type {t}")
    return tuple(1 if p == "?" else int(p) for p in mm.group(1).split("x") if p), mm.group(2)


def _parse_dense(body: str, shape, dtype):
    np_t = _NP[dtype]
    body = body.strip()
    n = int(np.prod(shape)) if shape else 1
    if body.startswith('"0x'):
        raw = bytes.fromhex(body[3:-1])
        return np.frombuffer(raw, dtype=np_t)[:n].reshape(shape).copy()
    is_float = dtype in ("f32", "bf16")
    if body.startswith("["):
        toks = re.findall(r"true|false|-?\d+(?:\.\d*)?(?:[eE][-+]?\d+)?", body)
        vals = [{"true": 1, "false": 0}[t] if t in ("true", "false") else (float(t) if is_float else int(t)) for t in toks]
        if dtype == "bf16":
            return _to_bf16_bits(vals).reshape(shape)
        return np.array(vals).astype(np_t).reshape(shape)
    v = {"true": 1, "false": 0}.get(body, None)
    if v is None:
        v = float(body) if is_float else int(body)
    if dtype == "bf16":
        return np.full(shape, _to_bf16_bits([v])[0], dtype=np.uint16)
    return np.full(shape, np.array(v).astype(np_t), dtype=np_t)


def _parse_attrs(text: str) -> dict:
    out = {}
    for k, v in re.findall(r"(\w+)\s*=\s*(array<i\d+:[^>]*>|\"[^\"]*\"|[-+\w\.]+(?:\s*:\s*\w+)?)", text):
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
                    try:
                        out[k] = float(tok)
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
        e = re.match(r"(%\w+)\s*=\s*tensor\.extract_slice\s+(%\w+)\[([^\]]*)\]\s*\[([^\]]*)\]\s*\[([^\]]*)\]\s*:\s*(tensor<[^>]*>)\s+to\s+(tensor<[^>]*>)", line)
        if e:
            ints = lambda t: [int(x) for x in re.findall(r"-?\d+", t)]
            if any(st != 1 for st in ints(e.group(5))):
                raise NotImplementedError("tensor.extract_slice with a stride")
            shape, dt = _parse_type(e.group(7))
            op = _Op("extract_slice", [vals[e.group(2)]], {"start": ints(e.group(3)), "size": ints(e.group(4))})
            op.result = _Val(e.group(1), shape, dt, op=op)
            vals[e.group(1)] = op.result
            if vals[e.group(2)].op is not None:
                vals[e.group(2)].op.users.append(op)
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


def _collapse(shape) -> tuple:
    """Tensors of the op list have at most four dimensions: the leading dimensions of a longer shape are merged
    (valid for the elementwise ops, the only ones the front end lets through with such shapes)."""
    shape = tuple(int(d) for d in shape)
    if len(shape) == 0:
        return (1,)  # a scalar tensor is one element
    if len(shape) <= 4:
        return shape
    return (int(np.prod(shape[:-3])),) + shape[-3:]


def build_graph(text: str) -> Graph:
    inputs, ops, returned = parse_module(text)
    g = Graph()
    env: dict[str, TensorRef] = {}
    for v in inputs:
        env[v.name] = g.input(_collapse(v.shape), graph_dtype(v.dtype))
    done: set[int] = set()
    deferred: dict[str, _Op] = {}  # i8->i32 rescales waiting for the add/sub/mul that absorbs them

    def get(v: _Val) -> TensorRef:
        """The op-list tensor of a TOSA value: an input or op result, a constant, or a rescale that was left
        for a fused consumer that did not come."""
        if v.name in env:
            return env[v.name]
        if v.const is not None:
            env[v.name] = g.const(np.ascontiguousarray(v.const).reshape(_collapse(v.shape) or (1,)).astype(_NP[v.dtype]).view(
                {"ui8": np.int8, "ui16": np.int16}.get(v.dtype, _NP[v.dtype])), graph_dtype(v.dtype))
            return env[v.name]
        if v.name in deferred:
            generic(deferred.pop(v.name))
            return env[v.name]
        raise NotImplementedError(f"value {v.name} has no producer the front end reads")

    def generic(op: _Op):
        """One op-list record per TOSA op, no fusion: the tensor ops outside the layer set."""
        n, res = op.name, op.result
        oshape, odt = _collapse(res.shape), graph_dtype(res.dtype)
        if n == "rescale":
            p = rescale_params(op)
            x = get(op.operands[0])
            mult, shift = (p["mult"], p["shift"]) if p["per_channel"] else (p["mult"][:1], p["shift"][:1])
            if not op.attrs.get("scale32", True):
                raise NotImplementedError("rescale with scale32 = false")
            izp, ozp = p["izp"], p["ozp"]
            if op.attrs.get("input_unsigned", False):
                izp &= (1 << (8 * np.dtype(_NP[op.operands[0].dtype]).itemsize)) - 1
            if op.attrs.get("output_unsigned", False):
                ozp &= (1 << (8 * np.dtype(_NP[res.dtype]).itemsize)) - 1
            env[res.name] = g.rescale(x, mult, shift, input_zp=izp, out_zp=ozp, double_round=p["double_round"], out_dtype=odt,
                                      input_unsigned=bool(op.attrs.get("input_unsigned", False)),
                                      output_unsigned=bool(op.attrs.get("output_unsigned", False)))
        elif n in ("exp", "log", "reciprocal", "rsqrt", "tanh", "sigmoid", "erf"):
            if op.operands[0].dtype not in ("f32", "bf16"):
                raise NotImplementedError(f"tosa.{n} on {op.operands[0].dtype}")
            env[res.name] = g.ew(n, get(op.operands[0]), out_dtype=odt)
        elif n == "matmul":
            a, b = op.operands[0], op.operands[1]
            if a.dtype not in ("bf16", "f32") or b.dtype != a.dtype or res.dtype not in ("bf16", "f32") or len(a.shape) != 3 or a.shape[0] != 1:
                raise NotImplementedError("tosa.matmul on these types")
            zps = [np.asarray(v.const).reshape(-1) for v in op.operands[2:4] if v.const is not None]
            if any(z.view(np.uint16 if a.dtype == "bf16" else np.uint32).any() for z in zps):
                raise NotImplementedError("float tosa.matmul with a zero point")
            y = g.matmul_f(g.reshape(get(a), a.shape[1:]), g.reshape(get(b), b.shape[1:]), out_dtype=odt)
            env[res.name] = g.reshape(y, oshape)
        elif n in ("abs", "bitwise_not", "logical_not", "clz", "ceil", "floor", "cast"):
            env[res.name] = g.ew(n, get(op.operands[0]), out_dtype=odt, bool_result=res.dtype == "i1" and n == "cast")
        elif n == "negate":
            izp = _scalar(op.operands[1]) if len(op.operands) > 1 else 0
            ozp = _scalar(op.operands[2]) if len(op.operands) > 2 else 0
            env[res.name] = g.ew("negate", get(op.operands[0]), out_dtype=odt, in_zp=izp, out_zp=ozp)
        elif n == "clamp":
            lo, hi = op.attrs["min_val"], op.attrs["max_val"]
            if res.dtype in ("f32", "bf16"):
                env[res.name] = g.ew("clamp", get(op.operands[0]), out_dtype=odt, fclamp=(float(lo), float(hi)))
            else:
                env[res.name] = g.ew("clamp", get(op.operands[0]), out_dtype=odt, clamp=(int(lo), int(hi)))
        elif n in ("add", "sub", "mul", "maximum", "minimum", "bitwise_and", "bitwise_or", "bitwise_xor", "logical_left_shift",
                   "arithmetic_right_shift", "equal", "greater", "greater_equal", "logical_and", "logical_or", "logical_xor"):
            a, b = get(op.operands[0]), get(op.operands[1])
            arg = 0
            if n == "mul" and len(op.operands) > 2:
                arg = _scalar(op.operands[2])
            if n == "arithmetic_right_shift":
                arg = 1 if op.attrs.get("round", False) else 0
            r = max(len(a.shape), len(b.shape))
            a = g.reshape(a, (1,) * (r - len(a.shape)) + a.shape) if len(a.shape) < r else a
            b = g.reshape(b, (1,) * (r - len(b.shape)) + b.shape) if len(b.shape) < r else b
            env[res.name] = g.ew(n, a, b, out_dtype=odt, arg=arg)
        elif n == "transpose":
            x = op.operands[0]
            perm = [int(v) for v in op.attrs["perms"]]
            if len(x.shape) > 6:
                raise NotImplementedError(f"rank {len(x.shape)} transpose")
            if len(x.shape) > 4:  # the stored tensor is the collapsed view of the same elements
                env[res.name] = g.permute(get(x), x.shape, perm, oshape)
            else:
                env[res.name] = g.transpose(get(x), perm)
        elif n in ("slice", "extract_slice"):
            x = op.operands[0]
            if len(x.shape) > 4:
                raise NotImplementedError(f"rank {len(x.shape)} slice")
            start = op.attrs["start"] if n == "extract_slice" else [int(v) for v in op.operands[1].const.reshape(-1)]
            size = op.attrs["size"] if n == "extract_slice" else [int(v) for v in op.operands[2].const.reshape(-1)]
            env[res.name] = g.slice(get(x), start, size)
        elif n == "pad":
            x = op.operands[0]
            if len(x.shape) > 4:
                raise NotImplementedError(f"rank {len(x.shape)} pad")
            amounts = [int(v) for v in op.operands[1].const.reshape(-1)]
            value = int(np.asarray(op.operands[2].const).reshape(-1).view(_NP[op.operands[2].dtype])[0]) if len(op.operands) > 2 else 0
            env[res.name] = g.pad(get(x), amounts[0::2], amounts[1::2], value)
        elif n == "concat":
            vals_ = [get(v) for v in op.operands]
            axis = int(op.attrs.get("axis", 0))
            if any(len(v.shape) > 4 for v in op.operands):
                raise NotImplementedError("rank > 4 concat")
            acc = vals_[0]
            for nxt in vals_[1:]:
                acc = g.concat_axis(acc, nxt, axis)
            env[res.name] = acc
        elif n in ("reduce_sum", "reduce_max", "reduce_min", "argmax"):
            x = op.operands[0]
            if len(x.shape) > 4:
                raise NotImplementedError(f"rank {len(x.shape)} reduction")
            fn = {"reduce_sum": "sum", "reduce_max": "max", "reduce_min": "min", "argmax": "argmax"}[n]
            t = g.reduce(fn, get(x), int(op.attrs["axis"]), keep_axis=n != "argmax", out_dtype=odt)
            env[res.name] = t if t.shape == oshape else g.reshape(t, oshape)
        elif n == "gather":
            vals_t, idx = op.operands
            if len(vals_t.shape) != 3 or idx.dtype != "i32":
                raise NotImplementedError("tosa.gather other than [N, K, C] values with i32 [N, W] indices")
            env[res.name] = g.gather(get(vals_t), get(idx))
        elif n == "scatter":
            vals_t, idx, upd = op.operands
            if len(vals_t.shape) != 3 or idx.dtype != "i32":
                raise NotImplementedError("tosa.scatter other than [N, K, C] values with i32 [N, W] indices")
            env[res.name] = g.scatter(get(vals_t), get(idx), get(upd))
        elif n == "identity":
            env[res.name] = g.reshape(get(op.operands[0]), oshape)
        elif n == "reshape":
            env[res.name] = g.reshape(get(op.operands[0]), oshape)
        elif n == "depthwise_conv2d" and op.operands[0].dtype in ("bf16", "f32"):
            x, w, bias, izp, wzp = op.operands
            if w.dtype != x.dtype or bias.dtype != x.dtype or res.dtype != x.dtype or len(x.shape) != 4 or len(w.shape) != 4:
                raise NotImplementedError("float tosa.depthwise_conv2d of mixed types")
            for z in (izp, wzp):
                if z.const is None or np.any(np.asarray(z.const)):
                    raise NotImplementedError("float tosa.depthwise_conv2d with a zero point")
            bt = get(bias)
            cm = int(w.shape[2]) * int(w.shape[3])
            if int(np.prod(bias.shape)) == 1 and cm != 1:  # a size-1 bias broadcasts over the channels
                if bias.const is None:
                    raise NotImplementedError("broadcast of a runtime bias")
                bt = g.const(np.repeat(np.asarray(get(bias).data).reshape(-1)[:1], cm), graph_dtype(x.dtype))
            pad = [int(v) for v in op.attrs.get("pad", [0] * 4)]
            env[res.name] = g.depthwise_conv2d_f(get(x), g.reshape(get(w), tuple(int(d) for d in w.shape)) if tuple(get(w).shape) != tuple(w.shape) else get(w),
                                                 bt, stride=[int(v) for v in op.attrs.get("stride", [1, 1])],
                                                 dilation=[int(v) for v in op.attrs.get("dilation", [1, 1])], pad=pad)
        elif n == "conv2d":
            # a 1x1 convolution whose weights are a second runtime tensor (a TFLite FULLY_CONNECTED / batch matmul of
            # two activations arrives like this): the matrix product of the pixels with the transposed weights
            x, w, bias, izp, wzp = op.operands
            if w.name not in env and w.name not in deferred:
                raise NotImplementedError("tosa.conv2d")
            if x.dtype != "i8" or w.dtype != "i8" or op.result.dtype != "i32" or tuple(w.shape[1:3]) != (1, 1) or \
                    [int(v) for v in op.attrs.get("stride", [1, 1])] != [1, 1] or any(int(v) for v in op.attrs.get("pad", [0] * 4)) or \
                    [int(v) for v in op.attrs.get("dilation", [1, 1])] != [1, 1]:
                raise NotImplementedError("tosa.conv2d with runtime weights other than 1x1 i8 x i8 -> i32")
            if bias.const is None or np.any(np.asarray(bias.const)):
                raise NotImplementedError("tosa.conv2d with runtime weights and a bias")
            K, OC = int(x.shape[-1]), int(w.shape[0])
            rows = int(np.prod(x.shape[:-1]))
            wt = g.transpose(g.reshape(get(w), (OC, K)), (1, 0))
            y = g.matmul_i32(g.reshape(get(x), (rows, K)), wt, a_zp=_scalar(izp), b_zp=_scalar(wzp))
            env[res.name] = g.reshape(y, oshape)
        else:
            raise NotImplementedError(f"tosa.{n}")

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

    def fused(op: _Op):
        """The layer-path forms (one record per fused chain); raises NotImplementedError when the op is not one."""
        n = op.name
        if n in ("conv2d", "depthwise_conv2d"):
            x, w, bias, izp, wzp = op.operands
            rs = only_user(op, "rescale")
            if rs is None or w.const is None:
                raise NotImplementedError(f"{n} without a constant weight and a following rescale")
            if n == "conv2d" and x.dtype == "i16" and w.dtype == "i8" and rs.result.dtype == "i16" and \
                    not rs.attrs.get("scale32", True) and "DOUBLE" not in str(rs.attrs.get("rounding_mode", "")):
                done.add(id(rs))
                p = rescale_params(rs)
                last, lo, hi = fold_clamp(rs, -32768, 32767)
                if p["izp"] != 0:
                    raise NotImplementedError("16-bit rescale of a convolution with an input zero point")
                mult, shift = (p["mult"], p["shift"]) if p["per_channel"] else (p["mult"][:1], p["shift"][:1])
                env[last.result.name] = g.conv2d_i16(get(x), w.const, bias.const.reshape(-1), mult, shift,
                                                     stride=tuple(op.attrs["stride"]), dilation=tuple(op.attrs["dilation"]),
                                                     pad=tuple(op.attrs["pad"]), input_zp=_scalar(izp), weight_zp=_scalar(wzp),
                                                     out_zp=p["ozp"], clamp=(lo, hi))
                return
            if x.dtype != "i8" or w.dtype != "i8" or rs.result.dtype != "i8":
                raise NotImplementedError(f"{n} on {x.dtype} activations")
            done.add(id(rs))
            p = rescale_params(rs)
            last, lo, hi = fold_clamp(rs)
            fn = g.conv2d if n == "conv2d" else g.depthwise_conv2d
            mult, shift = (p["mult"], p["shift"]) if p["per_channel"] else (p["mult"][:1], p["shift"][:1])
            y = fn(get(x), w.const, bias.const.reshape(-1), mult, shift, stride=tuple(op.attrs["stride"]),
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
                deferred[op.result.name] = op
                return  # consumed when the binary op is reached
            if src.dtype == "i32" and op.result.dtype == "i32" and src.op is not None and src.op.name == "rescale" and \
                    src.op.operands[0].dtype == "i8":
                users = list({id(u): u for u in op.users}.values())
                if len(users) != 1 or users[0].name not in ("add", "sub", "mul"):
                    raise NotImplementedError("i32->i32 rescale that does not feed add/sub/mul")
                deferred[op.result.name] = op
                return  # second input stage, consumed when the binary op is reached
            if src.dtype == "i8" and op.result.dtype == "i8":
                last, lo, hi = fold_clamp(op)
                mult, shift = (p["mult"], p["shift"]) if p["per_channel"] else (p["mult"][:1], p["shift"][:1])
                env[last.result.name] = g.rescale(get(src), mult, shift, input_zp=p["izp"], out_zp=p["ozp"],
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
            env[last.result.name] = fn(get(xa), get(xb), a_zp=za, a_ms=(ma, sa), b_zp=zb, b_ms=(mb, sb),
                                       out_ms=(int(po["mult"][0]), int(po["shift"][0])), out_zp=po["ozp"], clamp=(lo, hi),
                                       double_round=po["double_round"], a_lshift=la, b_lshift=lb)
        elif n == "table":
            if op.operands[0].dtype == "i16":
                env[op.result.name] = g.table16(get(op.operands[0]), op.operands[1].const.reshape(-1))
                return
            env[op.result.name] = g.table(get(op.operands[0]), op.operands[1].const.reshape(-1))
        elif n == "pad":
            mp = only_user(op, "max_pool2d")
            if mp is None:
                raise NotImplementedError("tosa.pad that does not feed max_pool2d")
            return
        elif n == "max_pool2d":
            src = op.operands[0]
            pad = list(op.attrs["pad"])
            pad_value = -32768 if src.dtype == "i16" else -128  # the type's lowest value: padding never wins
            if src.op is not None and src.op.name == "pad":
                amounts = src.op.operands[1].const.reshape(-1)  # [n0,n1,h0,h1,w0,w1,c0,c1]
                pad = [pad[0] + int(amounts[2]), pad[1] + int(amounts[3]), pad[2] + int(amounts[4]), pad[3] + int(amounts[5])]
                pad_value = _scalar(src.op.operands[2])
                src = src.op.operands[0]
            env[op.result.name] = g.maxpool2d(get(src), tuple(op.attrs["kernel"]), tuple(op.attrs["stride"]),
                                              tuple(pad), pad_value)
        elif n == "avg_pool2d":
            x, izp, ozp = op.operands
            env[op.result.name] = g.avg_pool2d(get(x), tuple(op.attrs["kernel"]), tuple(op.attrs["stride"]),
                                               tuple(op.attrs["pad"]), _scalar(izp), _scalar(ozp))
        elif n == "reshape":
            env[op.result.name] = g.reshape(get(op.operands[0]), _collapse(op.result.shape))
        elif n == "resize":
            x = op.operands[0]
            if op.attrs.get("mode") != "NEAREST_NEIGHBOR" or op.result.shape[1] != 2 * x.shape[1] or op.result.shape[2] != 2 * x.shape[2]:
                raise NotImplementedError("only 2x nearest-neighbour resize")
            env[op.result.name] = g.resize_nearest_2x(get(x))
        elif n == "concat":
            a, b = op.operands
            if int(op.attrs.get("axis", -1)) != len(a.shape) - 1:
                raise NotImplementedError("concat along a non-channel axis")
            one = (1 << 30, 30)
            env[op.result.name] = g.concat(get(a), get(b), a_zp=0, a_ms=one, b_zp=0, b_ms=one, out_zp=0)
        elif n == "matmul":
            a, b, azp, bzp = op.operands
            if a.dtype not in ("i8", "i16") or b.dtype != a.dtype or op.result.dtype not in ("i32", "i16") or \
                    len(a.shape) != 3 or a.shape[0] != 1:
                raise NotImplementedError("tosa.matmul other than one batch of i8 x i8 or i16 x i16 -> i32 or i16")
            y = g.matmul_i32(g.reshape(get(a), a.shape[1:]), g.reshape(get(b), b.shape[1:]), a_zp=_scalar(azp),
                             b_zp=_scalar(bzp), out_dtype=op.result.dtype)
            env[op.result.name] = g.reshape(y, op.result.shape)
        elif n == "clamp":
            x = op.operands[0]
            if x.dtype != "i8":
                raise NotImplementedError("clamp that does not follow a rescale")
            # on its own: the identity rescale (multiplier 2^30, shift 30 is exact) with the clamp range
            env[op.result.name] = g.rescale(get(x), np.array([1 << 30], np.int32), np.array([30], np.int8), input_zp=0,
                                            out_zp=0, clamp=(max(-128, int(op.attrs["min_val"])), min(127, int(op.attrs["max_val"]))),
                                            double_round=False)
        elif n == "identity":
            x = op.operands[0]
            env[op.result.name] = g.reshape(get(x), _collapse(x.shape))
        else:
            raise NotImplementedError(f"tosa.{n}")

    for op in ops:
        if id(op) in done:
            continue
        saved = set(done)
        mark = (len(g.ops), len(g.tensors), set(env))
        try:
            fused(op)
        except (NotImplementedError, ValueError):
            # not one of the fused layer forms: undo whatever the attempt emitted and read the op on its own
            done.clear()
            done.update(saved)
            deferred.pop(op.result.name, None)
            del g.ops[mark[0]:]
            del g.tensors[mark[1]:]
            for name in set(env) - mark[2]:
                del env[name]
            generic(op)
    for v in returned:
        t = get(v)
        if t.kind != ACTIVATION:
            # a value returned twice (or an input returned as it is): the further output is a copy of it
            t = g.reshape(t, t.shape)
        g.output(t)
    return g


def build_graph_from_file(path: str) -> Graph:
    with open(path) as f:
        return build_graph(f.read())
