"""Entry points with the names of qwix.pallas (qwix/pallas.py:37-65)."""

import functools

from qwix_b200 import qconfig
from qwix_b200.core import dot as _dot
from qwix_b200.core import dot_general as _dot_general
from qwix_b200.core import einsum as _einsum
from qwix_b200.core import pallas as _pallas
from qwix_b200.core import qarray as _qarray

__all__ = ['QArray', 'quantize', 'dequantize', 'get_current_rule', 'pallas_call', 'BlockSpec',
           'program_id', 'num_programs', 'dot_general', 'dot', 'einsum']

QArray = _qarray.QArray
quantize = _qarray.quantize_api
dequantize = _qarray.dequantize

get_current_rule = qconfig.get_current_rule
pallas_call = _pallas.pallas_call
BlockSpec = _pallas.BlockSpec
program_id = _pallas.program_id
num_programs = _pallas.num_programs

# The reference binds these to its per-K-tile loop implementation; here that loop is inside
# the GEMM kernel.
dot_general = _dot_general.loop_dot_general
dot = functools.partial(_dot.dot, _qwix_dot_general=dot_general)
einsum = functools.partial(_einsum.einsum, _qwix_dot_general=dot_general)
