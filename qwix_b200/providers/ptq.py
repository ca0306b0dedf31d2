"""Post-training-quantization provider: same policy as the reference, CUDA backends.

Restates the behaviour of qwix/_src/providers/boxed_param.py:37-499 and ptq.py:33-135.
The three injection points of the reference -- `_qarray_module`, `_dot_general_fn`,
`_einsum_fn` (boxed_param.py:92-107) -- default to this package's CUDA-backed modules, so
`PtqProvider(rules)` here equals `qwix.PtqProvider(rules, _qarray_module=..., ...)` there.
Weights are torch tensors owned by qwix_b200.nn modules instead of Flax variables.
"""

from __future__ import annotations

import dataclasses
import functools
from typing import Any, Callable, Generic, Mapping, Sequence, TypeVar

import torch

from qwix_b200 import _context
from qwix_b200 import fused
from qwix_b200 import qconfig
from qwix_b200.core import conv_general as conv_lib
from qwix_b200.core import dot as dot_lib
from qwix_b200.core import dot_general as dot_general_lib
from qwix_b200.core import einsum as einsum_lib
from qwix_b200.core import qarray

ArrayT = TypeVar('ArrayT')


@dataclasses.dataclass(frozen=True)
class WithAux(Generic[ArrayT]):
  """boxed_param.py:37-77 -- an array or QArray plus how it was (or is to be) quantized,
  so that quantize_params can quantize weights without running the model."""

  array: Any
  how: qarray.HowToQuantize

  value = property(lambda self: self.array)
  shape = property(lambda self: tuple(self.array.shape))
  ndim = property(lambda self: self.array.ndim)
  dtype = property(lambda self: self.array.dtype)

  def replace(self, **kw) -> 'WithAux':
    return dataclasses.replace(self, **kw)

  def astype(self, dtype) -> 'WithAux':
    a = self.array
    return self.replace(array=a.astype(dtype) if isinstance(a, qarray.QArray) else a.to(dtype))

  def reshape(self, *shape) -> 'WithAux':
    if len(shape) == 1 and not isinstance(shape[0], int):
      shape = tuple(shape[0])
    if tuple(self.shape) != tuple(shape):
      raise ValueError('Boxed weights should already have the target shape. Got'
                       f' {self.shape=} but {shape=} is requested.')
    return self


def _find_param(module, tensor) -> str | None:
  """Name of the parameter of `module` that `tensor` is (the role of
  flax_util.find_param, utils/flax_util.py:197-281: recognise a weight operand)."""
  if module is None or not isinstance(tensor, torch.Tensor):
    return None
  for name, p in module.named_parameters(recurse=False):
    if p is tensor or (p.data_ptr() == tensor.data_ptr() and p.shape == tensor.shape):
      return name
  return None


class BoxedParamProvider(qconfig.QuantizationProvider):
  """boxed_param.py:84-413 -- intercepts dot_general / einsum / dot of a running model."""

  def __init__(self, rules: Sequence[qconfig.QuantizationRule], *, disable_jit: bool = False,
               _qarray_module=qarray, _dot_general_fn=dot_general_lib.dot_general,
               _einsum_fn=einsum_lib.einsum,
               _conv_general_dilated_fn=conv_lib.conv_general_dilated):
    super().__init__(rules, disable_jit=disable_jit)
    self._qarray_module = _qarray_module
    self._dot_general_fn = _dot_general_fn
    self._einsum_fn = _einsum_fn
    self._conv_general_dilated_fn = _conv_general_dilated_fn

  def _prepare(self, lhs, rhs, rule, op_id, get_how):
    """Shared operand policy of boxed_param.py:137-168 / 204-235."""
    if isinstance(rhs, WithAux):  # weight, already quantized
      rhs = rhs.array
    elif weight_name := _find_param(_context.current_module(), rhs):  # weight, not yet
      rhs_how = get_how(for_lhs=False, qtype=rule.weight_qtype,
                        calibration_method=rule.weight_calibration_method)
      rhs = create_quantized_param(weight_name, rhs, rhs_how,
                                   _qarray_module=self._qarray_module).array
    elif rule.act_qtype is not None:  # activation on the right-hand side
      rhs_how = get_how(for_lhs=False, qtype=rule.act_qtype,
                        calibration_method=rule.act_calibration_method)
      rhs = quantize_act(rhs, rhs_how, rule, op_id + '_rhs',
                         _qarray_module=self._qarray_module)
    if rule.act_qtype is not None:
      lhs_how = get_how(for_lhs=True, qtype=rule.act_qtype,
                        calibration_method=rule.act_calibration_method)
      lhs = quantize_act(lhs, lhs_how, rule, op_id + '_lhs',
                         _qarray_module=self._qarray_module)
    elif isinstance(lhs, fused.LazyAct):  # weight-only rule: the activation stays floating
      lhs = lhs.materialize()
    return lhs, rhs

  def dot_general(self, lhs, rhs, dimension_numbers, precision=None,
                  preferred_element_type=None, *, out_sharding=None):
    """boxed_param.py:109-171."""
    rule, op_id = self._get_current_rule_and_op_id('dot_general')
    if rule is None or rule.weight_qtype is None:
      lhs, rhs = _plain(lhs), _plain(rhs)
      return dot_general_lib._plain_dot_general(lhs, rhs, dimension_numbers,
                                                preferred_element_type)
    get_how = functools.partial(dot_general_lib.get_how_to_quantize,
                                dimension_numbers=dimension_numbers,
                                ndims=(len(lhs.shape), len(rhs.shape)),
                                tile_size=rule.tile_size)
    lhs, rhs = self._prepare(lhs, rhs, rule, op_id, get_how)
    return self._dot_general_fn(lhs, rhs, dimension_numbers, out_sharding=out_sharding)

  def einsum(self, einsum_str: str, *operands, precision=None, preferred_element_type=None,
             out_sharding=None):
    """boxed_param.py:173-236."""
    rule, op_id = self._get_current_rule_and_op_id('einsum')
    if rule is None or rule.weight_qtype is None:
      return torch.einsum(einsum_str, *[_plain(o) for o in operands])
    if len(operands) != 2:
      raise ValueError(f'Unsupported einsum format: {einsum_str=} {operands=}')
    lhs, rhs = operands
    get_how = functools.partial(einsum_lib.get_how_to_quantize, einsum_str=einsum_str,
                                ndims=(len(lhs.shape), len(rhs.shape)),
                                tile_size=rule.tile_size)
    lhs, rhs = self._prepare(lhs, rhs, rule, op_id, get_how)
    return self._einsum_fn(einsum_str, lhs, rhs)

  def conv_general_dilated(self, lhs, rhs, window_strides, padding, lhs_dilation=None,
                           rhs_dilation=None, dimension_numbers=None, feature_group_count=1,
                           batch_group_count=1, precision=None, preferred_element_type=None,
                           out_sharding=None):
    """boxed_param.py:238-314 -- filter quantized per output channel (offline or at first use),
    input per image; the rule must give both the same qtype."""
    rule, op_id = self._get_current_rule_and_op_id('conv_general_dilated')
    kw = dict(lhs_dilation=lhs_dilation, rhs_dilation=rhs_dilation,
              dimension_numbers=dimension_numbers, feature_group_count=feature_group_count,
              batch_group_count=batch_group_count)
    if rule is None or rule.weight_qtype is None:
      return conv_lib.conv_general_dilated(_plain(lhs), _plain(rhs), window_strides, padding,
                                           preferred_element_type=preferred_element_type, **kw)
    rshape = rhs.array.qvalue.shape if isinstance(rhs, WithAux) else rhs.shape
    dn = conv_lib.conv_dimension_numbers(tuple(lhs.shape), tuple(rshape), dimension_numbers)
    kw['dimension_numbers'] = dn
    if isinstance(rhs, WithAux):
      rhs = rhs.array
    else:
      weight_name = _find_param(_context.current_module(), rhs)
      rhs_how = conv_lib.get_how_to_quantize(dimension_numbers=dn, for_lhs=False,
                                             qtype=rule.weight_qtype,
                                             calibration_method=rule.weight_calibration_method)
      rhs = create_quantized_param(weight_name, rhs, rhs_how,
                                   _qarray_module=self._qarray_module).array
    if rule.act_qtype != rule.weight_qtype:
      raise ValueError('conv_general_dilated requires same act_qtype and weight_qtype. Got:'
                       f' {rule.act_qtype=} {rule.weight_qtype=}')
    lhs_how = conv_lib.get_how_to_quantize(dimension_numbers=dn, for_lhs=True, qtype=rule.act_qtype,
                                           calibration_method=rule.act_calibration_method)
    lhs = quantize_act(_plain(lhs), lhs_how, rule, op_id + '_lhs', _qarray_module=self._qarray_module)
    return self._conv_general_dilated_fn(lhs, rhs, window_strides, padding, **kw)

  def dot(self, a, b, precision=None, preferred_element_type=None, out_sharding=None):
    """boxed_param.py:332-348."""
    return dot_lib.dot(a, b, precision=precision,
                       preferred_element_type=preferred_element_type,
                       out_sharding=out_sharding, _qwix_dot_general=self.dot_general)

  def asarray(self, a, dtype=None):
    """boxed_param.py:350-400 -- keep WithAux / QArray intact, cast their dequant dtype."""
    if isinstance(a, WithAux):
      return a.replace(array=self.asarray(a.array, dtype=dtype))
    if isinstance(a, qarray.QArray):
      return a.astype(dtype) if dtype is not None and a.dtype != dtype else a
    return torch.as_tensor(a, dtype=dtype)

  def get_intercept_map(self) -> Mapping[str, Callable]:
    """boxed_param.py:402-413 -- op name -> handler, as qwix_b200.ops dispatches."""
    return {'dot_general': self.dot_general, 'einsum': self.einsum, 'dot': self.dot,
            'conv_general_dilated': self.conv_general_dilated, 'asarray': self.asarray}


class PtqProvider(BoxedParamProvider):
  """ptq.py:33-49.  Weights may be handed over un-quantized: the first call of a module
  quantizes them in place; quantize_params does the same offline."""


def _plain(x):
  if isinstance(x, fused.LazyAct):
    return x.materialize()
  if isinstance(x, WithAux):
    x = x.array
  return qarray.dequantize(x) if isinstance(x, qarray.QArray) else x


def calibration_from_quant_stat(quant_stat: Mapping[str, Any]) -> dict:
  """averaging.py:67-98 (SimpleMovingAverage.get_calibration without a default): every
  `sum_of_<key>` divided by `count`, in the float32 the sums are kept in."""
  count = quant_stat['count']
  if int(count) == 0:
    raise ValueError('quant_stats is not initialized.')
  return {k[len('sum_of_'):]: v / count for k, v in quant_stat.items() if k.startswith('sum_of_')}


def quantize_act(array: torch.Tensor, how: qarray.HowToQuantize,
                 rule: qconfig.QuantizationRule, act_name: str, *,
                 _qarray_module=qarray) -> qarray.QArray:
  """boxed_param.py:416-455 -- dynamic range, or a static scale kept on the module.  A
  fused.LazyAct (an activation whose producing kernel can quantize on the way out) is asked
  for the QArray directly."""
  if isinstance(array, fused.LazyAct):
    if not rule.act_static_scale:
      return array.quantized(how, _qarray_module=_qarray_module)
    array = array.materialize()
  if not rule.act_static_scale:
    return _qarray_module.quantize(array, how)
  module = _context.current_module()
  scale_name, zp_name = act_name + '_scale', act_name + '_zero_point'
  box = getattr(module, scale_name, None) if module is not None else None
  if box is None:
    # Statistics gathered by a calibration or QAT run, kept on the module as
    # `quant_stats[act_name]`, are used once and removed (boxed_param.py:428-434).
    stats = getattr(module, 'quant_stats', None) if module is not None else None
    quant_stat = stats.pop(act_name, None) if isinstance(stats, dict) else None
    if quant_stat is not None:
      calibration = calibration_from_quant_stat(quant_stat)
    else:
      calibration = _qarray_module.calibrate(array, how)
      axes = [a for a in rule.act_batch_axes if a < array.ndim]
      calibration = {k: v.float().mean(dim=axes, keepdim=True).to(v.dtype)
                     for k, v in calibration.items()}
    scale, zp = _qarray_module.compute_scale_zero_point(calibration, how.qtype)
    box = WithAux(scale, how)
    if module is not None:
      setattr(module, scale_name, box)
      if zp is not None:
        setattr(module, zp_name, zp)
  else:
    zp = getattr(module, zp_name, None)
  return _qarray_module.quantize_with_scale_zero_point(array, how.qtype, box.array, zp)


def create_quantized_param(name: str, value: torch.Tensor, how: qarray.HowToQuantize, *,
                           _qarray_module=qarray) -> WithAux:
  """boxed_param.py:458-499 -- quantize a weight and store the boxed result on the module
  in place of the floating-point parameter."""
  boxed = WithAux(_qarray_module.quantize(value.detach(), how), how)
  module = _context.current_module()
  if module is not None and name in getattr(module, '_parameters', {}):
    del module._parameters[name]
    setattr(module, name, boxed)
  return boxed


def _flatten(tree: Mapping, prefix=()):
  for k, v in tree.items():
    if isinstance(v, Mapping):
      yield from _flatten(v, prefix + (k,))
    else:
      yield prefix + (k,), v


def _lookup(tree, path):
  for k in path:
    if isinstance(tree, Mapping):
      if k not in tree:
        return None
      tree = tree[k]
    else:
      tree = getattr(tree, k, None)
      if tree is None:
        return None
  return tree


def _unflatten(flat: Mapping[tuple, Any]) -> dict:
  out: dict = {}
  for path, v in flat.items():
    node = out
    for k in path[:-1]:
      node = node.setdefault(k, {})
    node[path[-1]] = v
  return out


def quantize_params(params: Any, abstract_quantized_params: Any, quant_stats: Any = None, *,
                    allow_extra_params: bool = False, _qarray_module=qarray) -> Any:
  """ptq.py:52-135 -- quantize a nested dict of floating-point weights.

  `abstract_quantized_params` is the param tree of the PTQ model (nested dict or the model
  itself); its WithAux leaves say how each weight is quantized and in which shape it is
  used.  Leaves without a WithAux template pass through.

  `quant_stats` (static-range quantization, ptq.py:106-129): a nested dict whose leaves are
  `{'count': n, 'sum_of_absmax': ...}` (or `sum_of_min` / `sum_of_max`) under the name of an
  activation, e.g. `{'Dense_0': {'dot_general0_lhs': {...}}}`.  Each becomes the static
  `<name>_scale` (and `<name>_zero_point`) of that activation; the qtype comes from the
  `<name>_scale` WithAux of the abstract tree.
  """
  out = {}
  for path, param in _flatten(params):
    if not isinstance(param, torch.Tensor):
      raise TypeError(f'params is not a pure dict of tensors: {type(param)}')
    template = _lookup(abstract_quantized_params, path)
    if template is None:
      if allow_extra_params:
        continue
      raise ValueError(f'{path} is not found in the abstract_quantized_params.')
    if isinstance(template, WithAux):
      param = param.reshape(template.shape)
      param = template.replace(array=_qarray_module.quantize(param, template.how))
    out[path] = param

  stat_paths = {path[:-1] for path, _ in _flatten(quant_stats or {})}
  for path in stat_paths:
    quant_stat = _lookup(quant_stats, path)
    if int(quant_stat['count']) == 0:
      raise ValueError(f'quant_stats is not initialized for {path}.')
    scale_path = (*path[:-1], path[-1] + '_scale')
    abs_scale = _lookup(abstract_quantized_params, scale_path)
    if not isinstance(abs_scale, WithAux):
      raise ValueError(f'{scale_path} is not a static scale of the abstract_quantized_params.')
    scale, zero_point = _qarray_module.compute_scale_zero_point(
        calibration_from_quant_stat(quant_stat), abs_scale.how.qtype)
    out[scale_path] = abs_scale.replace(array=scale)
    if zero_point is not None:
      out[(*path[:-1], path[-1] + '_zero_point')] = zero_point
  return _unflatten(out)
