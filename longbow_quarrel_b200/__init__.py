"""Import name of the package whose sources live in the folder `longbow-quarrel_b200/`.

A folder name with a hyphen cannot be imported, so this module stands in for it:
it points its package path at that folder and runs the folder's `__init__.py` as
its own body.  `import longbow_quarrel_b200.engine` therefore loads
`longbow-quarrel_b200/engine/`.
"""
from pathlib import Path as _Path

_SRC = _Path(__file__).resolve().parent.parent / "longbow-quarrel_b200"
__path__ = [str(_SRC)]
__file__ = str(_SRC / "__init__.py")
exec(compile((_SRC / "__init__.py").read_text(), __file__, "exec"))
