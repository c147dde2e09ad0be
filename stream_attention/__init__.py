"""``stream_attention`` import name for the B200-native decode path.

Code written against the StreamAttn reference imports ``stream_attention`` and its
sub-modules (``stream_attention.decode``, ``.engine``, ``.paged``, ``.backends.sm90``,
``.seed_selectors``, ``.seed_autotune``, ``.bucket_policy``, ``.telemetry`` and the kernel
launcher modules under ``.kernels``).  This package makes those import paths resolve to
``streamattn_b200``: each name below is the SAME module object as its implementation
(registered in ``sys.modules``), so classes compare equal across the two import names and
there is one copy of every piece of state.

Only the decode path is provided (reference ``stream_attention/__init__.py:69-125``).  The
training modules, the Gate-1 / fused-hybrid research routes and the profiler helper
``decode_cost_model_from_profile_rows`` are not part of this package.
"""

import importlib
import sys
import types

import streamattn_b200 as _impl

__version__ = _impl.__version__

# import path under stream_attention  ->  implementing module
_ALIASES = {
    "decode": "streamattn_b200.decode",
    "engine": "streamattn_b200.engine",
    "paged": "streamattn_b200.paged",
    "telemetry": "streamattn_b200.telemetry",
    "seed_selectors": "streamattn_b200.seed_selectors",
    "seed_autotune": "streamattn_b200.seed_autotune",
    "bucket_policy": "streamattn_b200.bucket_policy",
    "kv_update": "streamattn_b200.kv_update",
    "context_parallel": "streamattn_b200.context_parallel",
    # the reference's sm_90 backend package: the bound exact plan lives there
    "backends.sm90": "streamattn_b200.exact",
    "backends.sm90.transposed_gqa_exact": "streamattn_b200.exact",
    # kernel launcher modules (one implementation module serves all four names)
    "kernels.paged_exact_triton": "streamattn_b200.launchers",
    "kernels.gate0_exact_refresh_triton": "streamattn_b200.launchers",
    "kernels.gate0_seed_only_triton": "streamattn_b200.launchers",
    "kernels.qwen_o_proj_triton": "streamattn_b200.launchers",
}


def _namespace(name: str) -> types.ModuleType:
    module = types.ModuleType(name)
    module.__path__ = []  # a package with no files of its own
    sys.modules[name] = module
    return module


for _parent in ("backends", "kernels"):
    setattr(sys.modules[__name__], _parent, _namespace(f"{__name__}.{_parent}"))
for _path, _target in _ALIASES.items():
    _module = importlib.import_module(_target)
    sys.modules[f"{__name__}.{_path}"] = _module
    _owner_name, _, _leaf = _path.rpartition(".")
    _owner = sys.modules[f"{__name__}.{_owner_name}"] if _owner_name else sys.modules[__name__]
    setattr(_owner, _leaf, _module)

# Package-level names, as `from stream_attention import X` expects them.
for _name in _impl.__all__:
    globals()[_name] = getattr(_impl, _name)
decode = _impl.stream_attn_decode
# `import stream_attention.decode` made the attribute `decode` a module above; the reference
# resolves `stream_attention.decode` to the one-shot function (its __init__ rebinds the name
# after importing the sub-module), and so does this package.  `from stream_attention.decode
# import ...` still reaches the module through sys.modules.

__all__ = sorted(set(_impl.__all__) | {"decode"})
