"""The reference's own import paths, bound to this package.

Callers of the reference write

    import flydsl.compiler as flyc
    from kernels.gemm.preshuffle_gemm import compile_preshuffle_gemm
    from tests.utils import pertoken_quant, shuffle_weight

(tests/kernels/test_preshuffle_gemm.py:21,35,38 of the reference).  After

    import flydsl_b200.compat
    flydsl_b200.compat.install()

those lines resolve to the B200 implementation without a change to the calling
file: ``install`` registers aliases in ``sys.modules``; it puts nothing on disk
and refuses to shadow a real ``flydsl`` or ``kernels`` package that is already
imported.
"""

from __future__ import annotations

import importlib
import sys
import types

# reference module path -> module of this package that takes its place
ALIASES = {
    "flydsl.compiler": "flydsl_b200.compiler",
    "kernels.gemm.preshuffle_gemm": "flydsl_b200.kernels.gemm.preshuffle_gemm",
    "kernels.gemm.mxfp4_preshuffle": "flydsl_b200.kernels.gemm.mxfp4_preshuffle",
    "kernels.moe.moe_gemm_2stage": "flydsl_b200.kernels.moe.moe_gemm_2stage",
}


def install(force: bool = False) -> list[str]:
    """Register the aliases; returns the module names now served by this package."""
    done = []
    for ref_name, our_name in ALIASES.items():
        try:
            ours = importlib.import_module(our_name)
        except ModuleNotFoundError:
            continue
        parts = ref_name.split(".")
        for i in range(1, len(parts)):  # parent packages as empty namespace modules
            parent = ".".join(parts[:i])
            existing = sys.modules.get(parent)
            if existing is None:
                mod = types.ModuleType(parent)
                mod.__path__ = []  # a package: submodules resolve through sys.modules
                mod.__flydsl_b200_alias__ = True
                sys.modules[parent] = mod
            elif not getattr(existing, "__flydsl_b200_alias__", False) and not force:
                raise ImportError(f"a real '{parent}' package is already imported; refusing to shadow it")
        sys.modules[ref_name] = ours
        setattr(sys.modules[".".join(parts[:-1])], parts[-1], ours)
        for i in range(1, len(parts) - 1):
            setattr(sys.modules[".".join(parts[:i])], parts[i], sys.modules[".".join(parts[: i + 1])])
        done.append(ref_name)
    return done
