"""Importable alias of the ``aws-ofi-nccl_b200`` source directory.

The framework lives in a directory whose name contains hyphens (it mirrors the name of the
project it replaces), which Python cannot import directly.  This shim makes
``import aws_ofi_nccl_b200`` resolve to that directory.
"""
import os as _os

_real = _os.path.normpath(_os.path.join(_os.path.dirname(_os.path.abspath(__file__)), "..", "aws-ofi-nccl_b200"))
__path__ = [_real]
with open(_os.path.join(_real, "__init__.py")) as _f:
    exec(compile(_f.read(), _os.path.join(_real, "__init__.py"), "exec"))
del _f
