"""Switches of the package (mirror of ``src/flag_gems/config.py``).

In the reference ``use_c_extension`` routes operators to its C++ wrappers when the
optional extension was built and ``USE_C_EXTENSION=1``.  Here the C-ABI library is the
only implementation, so the native route is always on; ``aten_patch_list`` (ATen keys
taken over on the C++ side, which ``Register`` must skip) is empty because every ATen
override of this package is registered from Python.
"""
has_c_extension = True
use_c_extension = True
aten_patch_list: list = []
