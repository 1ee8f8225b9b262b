"""Device strings, as python/quabla/_devices.py:13-23 parses them.  Only CUDA
devices run here: there is no CPU path behind this package."""

from __future__ import annotations

from ._errors import UnsupportedOperationError


def parse_device(device: str | None) -> tuple[str, int]:
    if device is None or device == "cuda":
        return "cuda", 0
    if device == "cpu":
        return "cpu", 0
    if isinstance(device, str) and device.startswith("cuda:") and device[5:].isdigit():
        return "cuda", int(device[5:])
    raise ValueError(f"device must be None, 'cuda' or 'cuda:N', got {device!r}")


def require_device(device: str | None, op: str) -> tuple[str, int]:
    target, ordinal = parse_device(device)
    if target != "cuda":
        raise UnsupportedOperationError(
            f"{target} target is unavailable in this build: quabla_b200 runs on CUDA devices only and has no "
            "CPU fallback", op=op, device=device)
    return target, ordinal
