"""protobuf-to-json: convert a legacy TASO substitution collection (``graph_subst*.pb``) to the JSON rule format.

    python -m flexflow_train_b200.bin.protobuf_to_json graph_subst.pb rules.json

Counterpart of the reference tool (bin/protobuf-to-json/protobuf_to_json.cc, schema bin/protobuf-to-json/rules.proto).
The schema is six small proto2 messages of varint fields and nested messages, so the wire format is decoded
directly here -- no protobuf runtime or generated code is needed.  The JSON that comes out is what the legacy rule
loader of the substitution engine reads (``load_legacy_rules``).
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import Dict, List, Tuple

# Enumerators of the legacy file format, in file order (value = position).
OP_TYPES = ["OP_INPUT", "OP_WEIGHT", "OP_ANY", "OP_CONV2D", "OP_DROPOUT", "OP_LINEAR", "OP_POOL2D_MAX", "OP_POOL2D_AVG", "OP_RELU",
            "OP_SIGMOID", "OP_TANH", "OP_BATCHNORM", "OP_CONCAT", "OP_SPLIT", "OP_RESHAPE", "OP_TRANSPOSE", "OP_EW_ADD", "OP_EW_MUL",
            "OP_MATMUL", "OP_MUL", "OP_ENLARGE", "OP_MERGE_GCONV", "OP_CONSTANT_IMM", "OP_CONSTANT_ICONV", "OP_CONSTANT_ONE",
            "OP_CONSTANT_POOL", "OP_PARTITION", "OP_COMBINE", "OP_REPLICATE", "OP_REDUCE", "OP_EMBEDDING"]
PARAM_TYPES = ["PM_OP_TYPE", "PM_NUM_INPUTS", "PM_NUM_OUTPUTS", "PM_GROUP", "PM_KERNEL_H", "PM_KERNEL_W", "PM_STRIDE_H", "PM_STRIDE_W",
               "PM_PAD", "PM_ACTI", "PM_NUMDIM", "PM_AXIS", "PM_PERM", "PM_OUTSHUFFLE", "PM_MERGE_GCONV_COUNT", "PM_PARALLEL_DIM",
               "PM_PARALLEL_DEGREE"]
ACTIVATIONS = ["AC_MODE_NONE", "AC_MODE_SIGMOID", "AC_MODE_RELU", "AC_MODE_TANH"]
PADDINGS = ["PD_MODE_SAME", "PD_MODE_VALID"]


class WireError(ValueError):
    pass


def _varint(buf: bytes, pos: int) -> Tuple[int, int]:
    shift = result = 0
    while True:
        if pos >= len(buf):
            raise WireError("truncated varint")
        b = buf[pos]
        pos += 1
        result |= (b & 0x7F) << shift
        if not b & 0x80:
            return result, pos
        shift += 7
        if shift > 70:
            raise WireError("varint too long")


def _int32(v: int) -> int:
    """proto2 int32: negative values are stored as 64-bit two's complement varints."""
    v &= (1 << 64) - 1
    if v >= 1 << 63:
        v -= 1 << 64
    return int(v)


def _fields(buf: bytes) -> List[Tuple[int, int, object]]:
    """(field number, wire type, value) triples of one message."""
    out, pos = [], 0
    while pos < len(buf):
        key, pos = _varint(buf, pos)
        num, wt = key >> 3, key & 7
        if wt == 0:
            v, pos = _varint(buf, pos)
        elif wt == 2:
            n, pos = _varint(buf, pos)
            if pos + n > len(buf):
                raise WireError("truncated length-delimited field")
            v, pos = buf[pos:pos + n], pos + n
        elif wt == 1:
            v, pos = buf[pos:pos + 8], pos + 8
        elif wt == 5:
            v, pos = buf[pos:pos + 4], pos + 4
        else:
            raise WireError(f"unsupported wire type {wt}")
        out.append((num, wt, v))
    return out


def _name(table: List[str], v: int, what: str) -> str:
    if not 0 <= v < len(table):
        raise WireError(f"{what} {v} is outside the legacy enumeration")
    return table[v]


def _scalars(buf: bytes, names: Dict[int, str]) -> Dict[str, int]:
    return {names[n]: _int32(v) for n, wt, v in _fields(buf) if wt == 0 and n in names}


def _parameter(buf: bytes, symbolic_values: bool = False) -> dict:
    """Keys are always named; values stay integers as in the checked-in rule files unless `symbolic_values`
    asks for the activation / padding enumerator names."""
    f = _scalars(buf, {1: "key", 2: "value"})
    key = _name(PARAM_TYPES, f["key"], "parameter key")
    value = f["value"]
    if not symbolic_values:
        pass
    elif key == "PM_ACTI":
        value = _name(ACTIVATIONS, value, "activation")
    elif key == "PM_PAD":
        value = _name(PADDINGS, value, "padding mode")
    return {"_t": "Parameter", "key": key, "value": value}


def _operator(buf: bytes, symbolic_values: bool = False) -> dict:
    op = {"_t": "Operator", "input": [], "para": [], "type": None}
    for n, wt, v in _fields(buf):
        if n == 1 and wt == 0:
            op["type"] = _name(OP_TYPES, _int32(v), "operator type")
        elif n == 2 and wt == 2:
            op["input"].append(dict({"_t": "Tensor"}, **_scalars(v, {1: "opId", 2: "tsId"})))
        elif n == 3 and wt == 2:
            op["para"].append(_parameter(v, symbolic_values))
    return op


def _rule(buf: bytes, symbolic_values: bool = False) -> dict:
    r = {"_t": "Rule", "dstOp": [], "mappedOutput": [], "srcOp": []}
    for n, wt, v in _fields(buf):
        if wt != 2:
            continue
        if n == 1:
            r["srcOp"].append(_operator(v, symbolic_values))
        elif n == 2:
            r["dstOp"].append(_operator(v, symbolic_values))
        elif n == 3:
            r["mappedOutput"].append(dict({"_t": "MapOutput"}, **_scalars(v, {1: "srcOpId", 2: "dstOpId", 3: "srcTsId", 4: "dstTsId"})))
    return r


def decode_rule_collection(data: bytes, symbolic_values: bool = False) -> dict:
    rules = [_rule(v, symbolic_values) for n, wt, v in _fields(data) if n == 1 and wt == 2]
    for i, r in enumerate(rules):  # the JSON form names rules by their position in the collection
        r["name"] = f"taso_rule_{i}"
    return {"_t": "RuleCollection", "rule": rules}


# ---- encoder (used to produce test inputs and to convert JSON rule files back)
def _enc_varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        out.append(b | (0x80 if v else 0))
        if not v:
            return bytes(out)


def _enc_field(num: int, value) -> bytes:
    if isinstance(value, bytes):
        return _enc_varint(num << 3 | 2) + _enc_varint(len(value)) + value
    return _enc_varint(num << 3) + _enc_varint(int(value))


def encode_rule_collection(coll: dict) -> bytes:
    def op(o):
        b = _enc_field(1, OP_TYPES.index(o["type"]))
        for t in o["input"]:
            b += _enc_field(2, _enc_field(1, t["opId"]) + _enc_field(2, t["tsId"]))
        for p in o["para"]:
            v = p["value"]
            if p["key"] == "PM_ACTI" and isinstance(v, str):
                v = ACTIVATIONS.index(v)
            elif p["key"] == "PM_PAD" and isinstance(v, str):
                v = PADDINGS.index(v)
            b += _enc_field(3, _enc_field(1, PARAM_TYPES.index(p["key"])) + _enc_field(2, v))
        return b

    out = b""
    for r in coll["rule"]:
        rb = b"".join(_enc_field(1, op(o)) for o in r["srcOp"]) + b"".join(_enc_field(2, op(o)) for o in r["dstOp"])
        for m in r["mappedOutput"]:
            rb += _enc_field(3, _enc_field(1, m["srcOpId"]) + _enc_field(2, m["dstOpId"]) + _enc_field(3, m["srcTsId"]) +
                             _enc_field(4, m["dstTsId"]))
        out += _enc_field(1, rb)
    return out


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="protobuf-to-json", description="Convert a legacy substitution protobuf file to JSON.")
    p.add_argument("input", help="graph_subst*.pb")
    p.add_argument("output", nargs="?", help="JSON file (default: stdout)")
    p.add_argument("--indent", type=int, default=2)
    p.add_argument("--symbolic-values", action="store_true", help="write PM_ACTI / PM_PAD values as enumerator names")
    a = p.parse_args(argv)
    with open(a.input, "rb") as f:
        coll = decode_rule_collection(f.read(), a.symbolic_values)
    text = json.dumps(coll, indent=a.indent, sort_keys=True)
    if a.output:
        with open(a.output, "w") as f:
            f.write(text + "\n")
    else:
        sys.stdout.write(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
