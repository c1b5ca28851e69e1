"""B200-native convolution path for Theano graphs.

Importing the package registers the graph optimizers that swap the new ops in for the abstract
convolution ops (tag ``conv_b200``) when Theano is present: at once if the program has imported
Theano already, else if an importable Theano is found on the path.  Without Theano the
numpy-level calls of ``theano_b200.shim`` are still available.
"""
import importlib.util
import sys


def _register():
    if "theano" not in sys.modules:
        try:
            if importlib.util.find_spec("theano") is None:
                return False
        except (ImportError, ValueError):
            return False
    try:
        from . import opt  # noqa: F401  (registration is a side effect of the import)
    except Exception:      # a Theano that does not import in this interpreter
        return False
    return True


registered = _register()
