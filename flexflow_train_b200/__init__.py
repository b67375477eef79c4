"""flexflow_train_b200 -- a Blackwell-native auto-parallelizing training framework.

Layers (top to bottom): ``frontend`` (PyTorch fx / layer API) -> ``compiler`` (computation graph,
substitutions, Unity / MCMC strategy search; C++ core ``_ffcore``) -> ``runtime`` (lowering and
executors) -> ``parallel`` (NVLink peer-memory collectives fused with compute) -> ``ops`` (sm_100a
kernel library ``libffk.so``).
"""
__version__ = "0.1.0"

try:  # the C++ core is built in-tree by build.py
    from . import _ffcore  # noqa: F401
except ImportError as e:  # pragma: no cover
    raise ImportError("flexflow_train_b200._ffcore is not built: run `python build.py`") from e
