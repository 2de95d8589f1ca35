"""Body for a ``sitecustomize.py`` on PYTHONPATH: applies the FlashMLA patch in
every interpreter that starts, including the worker processes a serving
framework forks or spawns (reference: deepseek_v4_kernel/sitecustomize_hook.py).
Set DSV4_KERNEL_DISABLE=1 to skip.  A failure is reported on stderr and never
stops the interpreter."""
import os
import sys


def _apply() -> None:
    if os.environ.get("DSV4_KERNEL_DISABLE", "0") in ("1", "true", "yes"):
        return
    try:
        import deepseek_v4_kernel
        deepseek_v4_kernel.patch_flash_mla()
    except Exception as exc:  # noqa: BLE001
        sys.stderr.write(f"[deepseek_v4_kernel/sitecustomize] patch skipped: {exc}\n")


_apply()
