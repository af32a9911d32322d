"""Import alias for the package directory ``apus-deepseek-v4-flash_b200``.

The directory name carries hyphens, which Python cannot import directly, so
``import apus_b200`` loads that directory as the package ``apus_b200``.
"""
import importlib.util
import pathlib
import sys

_dir = pathlib.Path(__file__).resolve().parent / "apus-deepseek-v4-flash_b200"
_spec = importlib.util.spec_from_file_location(
    __name__, _dir / "__init__.py", submodule_search_locations=[str(_dir)])
_mod = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _mod
_spec.loader.exec_module(_mod)
