"""B200-native KVarN quantized paged KV-cache hot path (append, decode / verify / prefill attention).

The directory name is not a Python identifier; import it with importlib, e.g.

    import importlib.util, sys
    spec = importlib.util.spec_from_file_location("kvarn_b200", ".../ninfer-3080-iq3_s_b200/__init__.py",
                                                  submodule_search_locations=[".../ninfer-3080-iq3_s_b200"])
    mod = importlib.util.module_from_spec(spec); sys.modules["kvarn_b200"] = mod; spec.loader.exec_module(mod)

(`__graft_entry__.load_package()` at the repository root does exactly this.)
"""
from . import capi  # noqa: F401
from .build import build  # noqa: F401


def __getattr__(name):
    if name in ("sharded", "dump", "records"):
        import importlib

        return importlib.import_module(__name__ + "." + name)
    if name in ("KvarnLayer", "DecodeBatch", "merge_partials", "default_scale", "cache"):
        import importlib

        cache = importlib.import_module(__name__ + ".cache")
        return cache if name == "cache" else getattr(cache, name)
    raise AttributeError(name)
