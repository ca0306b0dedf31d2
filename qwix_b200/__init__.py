"""qwix_b200: the quantized-inference path of qwix on B200 (sm_100a) CUDA kernels.

Public names follow qwix/__init__.py:20-42.
"""

from qwix_b200.core.qarray import QArray, HowToQuantize, dequantize
from qwix_b200.core.qarray import quantize_api as quantize
from qwix_b200.core.dot_general import dot_general
from qwix_b200.core.einsum import einsum
from qwix_b200.core.dot import dot
from qwix_b200.core.ragged_dot import ragged_dot, ragged_dot_general
from qwix_b200.core.conv_general import conv_general_dilated
from qwix_b200.qconfig import QuantizationRule, QuantizationProvider, get_current_rule
from qwix_b200.providers.ptq import PtqProvider, WithAux, quantize_params
from qwix_b200.model import quantize_model

__all__ = ['QArray', 'HowToQuantize', 'quantize', 'dequantize', 'dot_general', 'einsum', 'dot',
           'ragged_dot', 'ragged_dot_general', 'conv_general_dilated',
           'QuantizationRule', 'QuantizationProvider', 'PtqProvider', 'WithAux',
           'quantize_model', 'quantize_params', 'get_current_rule']
