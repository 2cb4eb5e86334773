"""Opt-in read-back of the device-side error word of the look-back scans.

The S1/S2 look-back kernel bounds every wait on another tile; a wait that runs out records
``B200_ERR_TIMEOUT`` at the head of that launch's workspace and the kernel finishes with a zero
carry instead of hanging.  Reading the word back costs a stream synchronisation, so the ops never
do it on their own.  A caller that wants the check switches tracking on, which makes the launchers
remember the most recent workspace per device, and calls ``check_status()`` between steps::

    tsfast_b200.track_status(True)
    ...                       # training / inference steps
    tsfast_b200.check_status()  # raises RuntimeError if a launch since the last check timed out

With tracking off (the default) no workspace outlives its call.
"""

from __future__ import annotations

import torch

from . import _lib

__all__ = ["track_status", "check_status"]

_tracking = False
_recent: dict[int, torch.Tensor] = {}


def track_status(on: bool = True) -> None:
    """Start or stop remembering the latest look-back workspace of each device."""
    global _tracking
    _tracking = bool(on)
    if not _tracking:
        _recent.clear()


def remember(ws: torch.Tensor) -> None:
    """Called by the launchers after a launch that used ``ws`` (no-op unless tracking is on)."""
    if _tracking:
        _recent[ws.device.index or 0] = ws


def check_status(device=None) -> None:
    """Synchronise and raise if the latest tracked launch on ``device`` (default: all) recorded an error."""
    if not _tracking:
        raise RuntimeError("status tracking is off: call tsfast_b200.track_status(True) before the launches to check")
    wanted = None if device is None else (torch.device(device).index or 0)
    for index, ws in list(_recent.items()):
        if wanted is not None and index != wanted:
            continue
        code = int(_lib.lib().b200_workspace_status(_lib.ptr(ws), _lib.stream_ptr(ws.device)))
        if code != 0:
            _lib.check(code, f"a look-back scan on cuda:{index}")
