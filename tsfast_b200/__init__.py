"""tsfast_b200: B200-native (sm_100a) recurrent-scan kernels behind tsfast's scan interfaces.

Public surface:

* ``diagonal_recurrence`` / ``selective_recurrence`` – the scan functions, same signatures as
  ``tsfast.models._core.scan``;
* ``scan_backends.diagonal_b200`` / ``selective_b200`` – backend modules speaking tsfast's
  ``supports/forward/backward`` protocol;
* ``install()`` / ``uninstall()`` – plug those modules into an importable tsfast so that its LRU,
  S5, Mamba and dynoNet modules dispatch to these kernels;
* ``proj_b200`` / ``accelerate_linears()`` – the projections around the scans on the tensor cores;
* ``track_status()`` / ``check_status()`` – opt-in read-back of the look-back kernels' device-side
  error word between steps.

Everything runs through ``libb200scan.so`` (``python -m tsfast_b200.build``); nothing here falls
back to PyTorch or the CPU.
"""

from . import allpole_b200, conv_b200, dynonet_b200, glue_b200, lru_b200, mamba_b200, prologue_b200, proj_b200
from .scan import diagonal_recurrence, selective_recurrence
from .install import accelerate_linears, install, restore_linears, uninstall
from .status import check_status, track_status

__all__ = ["diagonal_recurrence", "selective_recurrence", "install", "uninstall", "accelerate_linears", "restore_linears",
           "track_status", "check_status"]
__version__ = "0.1.0"
