"""Exceptions that mirror the reference's error enums (crates/bobcat/src/error.rs:10-97 and
crates/bobcat-metal/src/backend.rs:163-298), one class per status code of the C ABI."""

from __future__ import annotations


class BobcatError(Exception):
    status = -1


def _make(name: str, status: int) -> type:
    cls = type(name, (BobcatError,), {"status": status})
    return cls


Io = _make("Io", 1)
Gguf = _make("Gguf", 2)
Metadata = _make("Metadata", 3)
Architecture = _make("Architecture", 4)
Hyperparameters = _make("Hyperparameters", 5)
OddHeadDim = _make("OddHeadDim", 6)
MissingTensor = _make("MissingTensor", 7)
TensorShape = _make("TensorShape", 8)
TensorType = _make("TensorType", 9)
KvHeads = _make("KvHeads", 10)
Token = _make("Token", 11)
ContextFull = _make("ContextFull", 12)
Argument = _make("Argument", 13)
Unsupported = _make("Unsupported", 14)
NoDevice = _make("NoDevice", 20)
Allocation = _make("Allocation", 21)
NotRecording = _make("NotRecording", 22)
AlreadyRecording = _make("AlreadyRecording", 23)
OutOfBounds = _make("OutOfBounds", 24)
ForeignBuffer = _make("ForeignBuffer", 25)
Busy = _make("Busy", 26)
AttentionLimits = _make("AttentionLimits", 27)
GateShape = _make("GateShape", 28)
NoFusedConv = _make("NoFusedConv", 29)
NoExpansion = _make("NoExpansion", 30)
NoExperts = _make("NoExperts", 31)
DeltaNetLimits = _make("DeltaNetLimits", 32)
ExpertLimits = _make("ExpertLimits", 33)
Execution = _make("Execution", 34)

BY_STATUS = {cls.status: cls for cls in list(globals().values()) if isinstance(cls, type) and issubclass(cls, BobcatError) and cls is not BobcatError}


def check(status: int, lib) -> None:
    """Raise the exception for a non-zero status, with the library's message."""
    if status == 0:
        return
    message = lib.bc_last_error().decode("utf-8", "replace")
    raise BY_STATUS.get(status, BobcatError)(message)
