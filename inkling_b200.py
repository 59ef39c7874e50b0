"""Import alias: `import inkling_b200` loads the package that lives in the directory
`inkling-vs-quad-rtx-3090s_b200/` (a name Python cannot import directly)."""
import importlib.util
import sys
from pathlib import Path

_root = Path(__file__).resolve().parent / "inkling-vs-quad-rtx-3090s_b200"
_spec = importlib.util.spec_from_file_location(__name__, _root / "__init__.py",
                                               submodule_search_locations=[str(_root)])
_module = importlib.util.module_from_spec(_spec)
sys.modules[__name__] = _module
_spec.loader.exec_module(_module)
