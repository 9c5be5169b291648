"""Scalar event files that TensorBoard reads, written without the ``tensorboard`` / ``tensorflow`` packages.

An event file is a sequence of records ``[uint64 length][masked crc32c of the length][payload][masked crc32c of the
payload]``; a payload is a serialised ``Event`` message (``wall_time`` field 1 double, ``step`` field 2 varint,
``file_version`` field 3 string or ``summary`` field 5), a ``Summary`` holds repeated ``Value`` messages (field 1) with
``tag`` (field 1 string) and ``simple_value`` (field 2 float).  The few message shapes needed are encoded by hand.

The reference gets this through the Hugging Face trainer's ``report_to: tensorboard`` integration
(``hparams/training_args.py``); :class:`TensorBoardCallback` is this package's counterpart."""
from __future__ import annotations

import os
import socket
import struct
import time
from typing import Dict, Iterator, List, Tuple

_CRC_TABLE: List[int] = []


def _table() -> List[int]:
    if not _CRC_TABLE:
        for n in range(256):
            c = n
            for _ in range(8):
                c = (c >> 1) ^ 0x82F63B78 if c & 1 else c >> 1          # Castagnoli polynomial, reflected
            _CRC_TABLE.append(c)
    return _CRC_TABLE


def crc32c(data: bytes) -> int:
    t, c = _table(), 0xFFFFFFFF
    for b in data:
        c = t[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def masked_crc(data: bytes) -> int:
    c = crc32c(data)
    return ((((c >> 15) | (c << 17)) & 0xFFFFFFFF) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(n: int) -> bytes:
    out = bytearray()
    n &= (1 << 64) - 1
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _field_bytes(number: int, payload: bytes) -> bytes:
    return _varint(number << 3 | 2) + _varint(len(payload)) + payload


def encode_scalar_event(tag: str, value: float, step: int, wall_time: float) -> bytes:
    val = _field_bytes(1, tag.encode()) + _varint(2 << 3 | 5) + struct.pack("<f", float(value))
    summary = _field_bytes(1, val)
    return _varint(1 << 3 | 1) + struct.pack("<d", wall_time) + _varint(2 << 3 | 0) + _varint(step) + \
        _field_bytes(5, summary)


def _record(payload: bytes) -> bytes:
    head = struct.pack("<Q", len(payload))
    return head + struct.pack("<I", masked_crc(head)) + payload + struct.pack("<I", masked_crc(payload))


class EventWriter:
    def __init__(self, log_dir: str):
        os.makedirs(log_dir, exist_ok=True)
        self.path = os.path.join(log_dir, f"events.out.tfevents.{int(time.time())}.{socket.gethostname()}.{os.getpid()}")
        self._f = open(self.path, "ab")
        version = _varint(1 << 3 | 1) + struct.pack("<d", time.time()) + _field_bytes(3, b"brain.Event:2")
        self._f.write(_record(version))
        self._f.flush()

    def add_scalar(self, tag: str, value: float, step: int) -> None:
        self._f.write(_record(encode_scalar_event(tag, value, step, time.time())))

    def add_scalars(self, values: Dict[str, float], step: int) -> None:
        for k, v in values.items():
            self.add_scalar(k, v, step)
        self._f.flush()

    def close(self) -> None:
        if not self._f.closed:
            self._f.close()


def read_scalars(path: str) -> Iterator[Tuple[str, float, int]]:
    """``(tag, value, step)`` of every scalar record; checks both checksums of every record (used by the tests and
    handy for reading a log without TensorBoard)."""
    with open(path, "rb") as f:
        data = f.read()
    pos = 0

    def varint(buf: bytes, i: int) -> Tuple[int, int]:
        n = shift = 0
        while True:
            b = buf[i]
            i += 1
            n |= (b & 0x7F) << shift
            shift += 7
            if not b & 0x80:
                return n, i

    def fields(buf: bytes) -> Iterator[Tuple[int, int, object]]:
        i = 0
        while i < len(buf):
            key, i = varint(buf, i)
            num, wire = key >> 3, key & 7
            if wire == 0:
                v, i = varint(buf, i)
            elif wire == 1:
                v, i = buf[i:i + 8], i + 8
            elif wire == 5:
                v, i = buf[i:i + 4], i + 4
            else:
                n, i = varint(buf, i)
                v, i = buf[i:i + n], i + n
            yield num, wire, v

    while pos < len(data):
        head = data[pos:pos + 8]
        (n,) = struct.unpack("<Q", head)
        if struct.unpack("<I", data[pos + 8:pos + 12])[0] != masked_crc(head):
            raise ValueError(f"{path}: bad length checksum at byte {pos}")
        payload = data[pos + 12:pos + 12 + n]
        if struct.unpack("<I", data[pos + 12 + n:pos + 16 + n])[0] != masked_crc(payload):
            raise ValueError(f"{path}: bad payload checksum at byte {pos}")
        pos += 16 + n
        step, summary = 0, None
        for num, _, v in fields(payload):
            if num == 2:
                step = v
            elif num == 5:
                summary = v
        if summary is None:
            continue
        for num, _, val in fields(summary):
            if num != 1:
                continue
            tag, x = "", None
            for fn, _, fv in fields(val):
                if fn == 1:
                    tag = fv.decode()
                elif fn == 2:
                    (x,) = struct.unpack("<f", fv)
            if x is not None:
                yield tag, x, step


class TensorBoardCallback:
    """Trainer callback: the scalars of every logged step go to ``<output_dir>/runs``."""

    def __init__(self, output_dir: str):
        self.dir = os.path.join(output_dir, "runs")
        self.writer = None
        self._last = -1

    def __call__(self, trainer) -> None:
        if trainer.rank != 0 or trainer.global_step == self._last:
            return
        loss = getattr(trainer, "_last_loss", None)
        steps = trainer.args.logging_steps
        if loss is None or not steps or trainer.global_step % steps:
            return
        if self.writer is None:
            self.writer = EventWriter(self.dir)
        self._last = trainer.global_step
        self.writer.add_scalars({"train/loss": loss, "train/learning_rate": getattr(trainer, "_last_lr", 0.0),
                                 "train/tokens_seen": float(getattr(trainer, "tokens_seen", 0))}, trainer.global_step)

    def on_train_end(self, trainer) -> None:
        if self.writer is not None:
            self.writer.close()
