"""ATen override registration (mirror of ``src/flag_gems/runtime/register.py:5-61``).

``Register`` takes ``(aten key, python function)`` pairs, drops the functions whose
``__name__`` the user listed in ``unused`` and the keys already patched natively, then
installs the rest on dispatch key ``CUDA`` of the given ``torch.library.Library``.
"""
from __future__ import annotations


class Register:
    reg_key = "CUDA"

    def __init__(self, config, user_unused_ops_list=None, cpp_patched_ops_list=None, lib=None):
        self.lib = lib
        self.all_ops = []
        self.unused_ops = list(user_unused_ops_list or [])
        self.cpp_patched_ops_list = set(cpp_patched_ops_list or [])
        self.config = [
            item for item in config
            if item[1].__name__ not in self.unused_ops and item[0] not in self.cpp_patched_ops_list
        ]
        self.for_each()

    def register_impl(self, key, fn):
        self.all_ops.append(key)
        self.lib.impl(key, fn, self.reg_key)

    def for_each(self):
        try:
            for key, func in self.config:
                self.register_impl(key, func)
        except Exception as e:  # same contract as runtime/error.py:12-15
            raise RuntimeError(e) from e

    def get_all_ops(self):
        return self.all_ops

    def get_unused_ops(self):
        return self.unused_ops

    def get_vendor_name(self):
        return "nvidia"

    def get_current_device(self):
        return "cuda"
