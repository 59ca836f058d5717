"""Import name of the library.  The sources live in the folder ``llm-inference-cpp_b200``
beside this one, whose name is not a Python identifier; this package maps itself onto it."""
import os as _os

__path__.insert(0, _os.path.join(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))),
                                 "llm-inference-cpp_b200"))
with open(_os.path.join(__path__[0], "__init__.py"), encoding="utf-8") as _f:
    exec(compile(_f.read(), _os.path.join(__path__[0], "__init__.py"), "exec"))
