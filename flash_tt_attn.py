"""``from flash_tt_attn import attention`` from the repository root, as in the reference's
example_usage.py: loads flash-triangle-attention_b200/flash_tt_attn.py under this name."""
import importlib.util
import os
import sys

_pkg = os.path.join(os.path.dirname(os.path.abspath(__file__)), "flash-triangle-attention_b200")
if _pkg not in sys.path:
    sys.path.insert(0, _pkg)
_spec = importlib.util.spec_from_file_location(__name__, os.path.join(_pkg, "flash_tt_attn.py"))
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
