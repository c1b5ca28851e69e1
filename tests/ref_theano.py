"""Test-side name of the reference import glue (it lives with the other checker code)."""
from oracle.ref_theano import *  # noqa: F401,F403
from oracle.ref_theano import REF_ROOT, available, import_theano  # noqa: F401
