"""proto3 wire format of REEF's six RPC messages, written by hand.

The reference describes its request API in ``src/reef/protos/reef.proto`` (service ``reef.rpc.REEFService``,
lines 5-23; messages lines 25-80) and compiles it with protoc + the gRPC C++ plugin.  Neither is needed to
speak it: every field is a bool, an int32/int64 (varint, wire type 0) or a string (length-delimited, wire
type 2), so the twelve messages are a table of (field number, name, kind) and forty lines of codec.
Default values (false, 0, "") are not written, as proto3 prescribes; unknown fields are skipped when read.
"""
from __future__ import annotations

from dataclasses import dataclass, field

BOOL, INT32, INT64, STRING = "bool", "int32", "int64", "string"

SERVICE = "reef.rpc.REEFService"

# message name -> [(field number, field name, kind)]   (reference: reef.proto, line of each message in brackets)
SCHEMAS = {
    "LoadModelRequest": [(1, "dir", STRING), (2, "name", STRING), (3, "qid", INT32)],   # [25]
    "LoadModelReply": [(1, "succ", BOOL), (2, "mid", INT32)],                           # [31]
    "SetPriorityRequest": [(1, "rt", BOOL)],                                             # [36]
    "SetPriorityReply": [(1, "succ", BOOL), (2, "qid", INT32)],                          # [40]
    "RegisterBlobRequest": [(1, "mid", INT32), (2, "name", STRING)],                     # [45]
    "RegisterBlobReply": [(1, "succ", BOOL), (2, "key", STRING), (3, "size", INT64)],    # [50]
    "GetBlobRequest": [(1, "key", STRING)],                                              # [56]
    "GetBlobReply": [(1, "succ", BOOL)],                                                 # [60]
    "SetBlobRequest": [(1, "key", STRING)],                                              # [64]
    "SetBlobReply": [(1, "succ", BOOL)],                                                 # [68]
    "InferRequest": [(1, "mid", INT32), (2, "async", BOOL)],                             # [72]
    "InferReply": [(1, "succ", BOOL), (2, "tid", INT32)],                                # [77]
}

# rpc name -> (request message, reply message)   (reference: reef.proto:5-23)
METHODS = {
    "LoadModel": ("LoadModelRequest", "LoadModelReply"),
    "SetPriority": ("SetPriorityRequest", "SetPriorityReply"),
    "RegisterBlob": ("RegisterBlobRequest", "RegisterBlobReply"),
    "GetBlob": ("GetBlobRequest", "GetBlobReply"),
    "SetBlob": ("SetBlobRequest", "SetBlobReply"),
    "Infer": ("InferRequest", "InferReply"),
}


def _varint(v: int) -> bytes:
    if v < 0:
        v += 1 << 64            # negative int32/int64 are sign-extended to ten bytes
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _read_varint(buf: bytes, pos: int):
    shift = v = 0
    while True:
        if pos >= len(buf):
            raise ValueError("truncated varint")
        b = buf[pos]
        pos += 1
        v |= (b & 0x7F) << shift
        if not b & 0x80:
            return v, pos
        shift += 7
        if shift > 63:
            raise ValueError("varint longer than ten bytes")


@dataclass
class Message:
    """One message instance: ``kind`` names its schema, ``f`` holds the fields that are set."""
    kind: str
    f: dict = field(default_factory=dict)

    def __getattr__(self, name):
        for _, fname, fkind in SCHEMAS[self.__dict__["kind"]]:
            if fname == name:
                return self.__dict__["f"].get(name, "" if fkind == STRING else (False if fkind == BOOL else 0))
        raise AttributeError(name)


def make(kind: str, **fields) -> Message:
    known = {n for _, n, _ in SCHEMAS[kind]}
    for k in fields:
        if k not in known:
            raise KeyError(f"{kind} has no field {k}")
    return Message(kind, dict(fields))


def encode(msg: Message) -> bytes:
    out = bytearray()
    for num, name, kind in SCHEMAS[msg.kind]:
        v = msg.f.get(name)
        if kind == STRING:
            if v:
                raw = v.encode()
                out += _varint(num << 3 | 2) + _varint(len(raw)) + raw
        elif kind == BOOL:
            if v:
                out += _varint(num << 3) + b"\x01"
        else:
            if v:
                out += _varint(num << 3) + _varint(int(v))
    return bytes(out)


def decode(kind: str, buf: bytes) -> Message:
    by_num = {num: (name, k) for num, name, k in SCHEMAS[kind]}
    msg = Message(kind, {})
    pos = 0
    while pos < len(buf):
        tag, pos = _read_varint(buf, pos)
        num, wt = tag >> 3, tag & 7
        if wt == 0:
            v, pos = _read_varint(buf, pos)
        elif wt == 2:
            n, pos = _read_varint(buf, pos)
            if pos + n > len(buf):
                raise ValueError("truncated length-delimited field")
            v, pos = buf[pos:pos + n], pos + n
        elif wt == 1:
            v, pos = buf[pos:pos + 8], pos + 8
        elif wt == 5:
            v, pos = buf[pos:pos + 4], pos + 4
        else:
            raise ValueError(f"unsupported wire type {wt}")
        if num not in by_num:
            continue
        name, k = by_num[num]
        if k == STRING:
            if wt != 2:
                raise ValueError(f"{kind}.{name}: expected a length-delimited field")
            msg.f[name] = bytes(v).decode()
        else:
            if wt != 0:
                raise ValueError(f"{kind}.{name}: expected a varint")
            if k == BOOL:
                msg.f[name] = bool(v)
            else:
                v &= (1 << 64) - 1
                if v >= 1 << 63:
                    v -= 1 << 64
                if k == INT32:
                    v = ((v + (1 << 31)) % (1 << 32)) - (1 << 31)
                msg.f[name] = v
    return msg
