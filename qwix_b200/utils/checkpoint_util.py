"""Pre-quantized checkpoints: load codes and scales that were quantized elsewhere into a PTQ
model, derive the rules they imply, and move such trees to and from disk.

The host logic of qwix/_src/utils/checkpoint_util.py:383-587 for this backend's models
(nested dicts of torch tensors and WithAux / QArray leaves instead of NNX state):

  process_prequantized_params   checkpoint leaf x template leaf -> the leaf to install
                                (:383-501; the three cases of :446-487)
  restore_quantization_rules    one rule per quantized module of a checkpoint (:504-587)
  save_prequantized / load_prequantized
                                a safetensors file per tree; int4 codes travel packed two per
                                byte, low nibble = even index (the layout of the C ABI)

Dequantization of a quantized checkpoint leaf for a floating-point template (case 2) runs on
the device through qwx_dequantize.
"""

from __future__ import annotations

import json
import logging
from typing import Any, Mapping

import torch

from qwix_b200 import qconfig
from qwix_b200.core import numerics
from qwix_b200.core import qarray
from qwix_b200.providers import ptq

_LEAF_NAMES = frozenset({'qvalue', 'scale', 'zero_point'})
_LEAF_EXTRAS = frozenset({'qtype'})   # rides along in trees made by this module
_DEFAULT_ACT_QTYPE = object()
logger = logging.getLogger(__name__)


def _is_quantized_leaf(x) -> bool:
  """checkpoint_util.py:31-45 -- a dict with a 'qvalue' key is one pre-quantized weight."""
  return isinstance(x, Mapping) and 'qvalue' in x


def _flatten(tree: Mapping, prefix=()):
  for k, v in tree.items():
    if isinstance(v, Mapping) and not _is_quantized_leaf(v):
      yield from _flatten(v, prefix + (k,))
    else:
      yield prefix + (k,), v


def _unflatten(flat: Mapping[tuple, Any]) -> dict:
  out: dict = {}
  for path, v in flat.items():
    node = out
    for k in path[:-1]:
      node = node.setdefault(k, {})
    node[path[-1]] = v
  return out


def _template_at(template: Any, path):
  """The template leaf at `path`; a trailing 'array' component (the WithAux field name that
  NNX state paths carry) is optional (checkpoint_util.py:352-380)."""
  if hasattr(template, 'params') and callable(template.params):
    template = template.params()
  elif isinstance(template, torch.nn.Module):
    from qwix_b200 import model as model_lib
    template = model_lib.get_params(template)
  for cand in (path, path[:-1] if path and path[-1] == 'array' else None):
    if cand is None:
      continue
    node = template
    for k in cand:
      if isinstance(node, Mapping) and k in node:
        node = node[k]
      else:
        node = None
        break
    if node is not None:
      return cand, node
  return path, None


def _validate(leaf: Any, path) -> None:
  """checkpoint_util.py:55-92."""
  if not isinstance(leaf, Mapping):
    raise ValueError(f'{path} is quantized in the template_params. Expected a dict containing'
                     ' qvalue/scale leaves.')
  extra = set(leaf) - _LEAF_NAMES - _LEAF_EXTRAS
  if extra:
    raise ValueError(f'{path} has unsupported quantized leaves {sorted(extra)}. Expected only'
                     f' {sorted(_LEAF_NAMES)}.')
  if 'qvalue' not in leaf or 'scale' not in leaf:
    raise ValueError(f'{path} is missing required "qvalue" or "scale" in pre-quantized'
                     f' dictionary. Found keys: {list(leaf.keys())}')


def _coerce(value: torch.Tensor, like: torch.Tensor, path, *, allow_broadcast=False,
            what='') -> torch.Tensor:
  """Shape, dtype and device of the template leaf (checkpoint_util.py:155-209): shapes must
  agree; scales and zero points may additionally be given with their size-1 axes dropped."""
  value = torch.as_tensor(value)
  if tuple(value.shape) != tuple(like.shape):
    if allow_broadcast and value.numel() == like.numel():
      value = value.reshape(like.shape)
    else:
      raise ValueError(f'{path}: {what} has shape {tuple(value.shape)}, the template expects'
                       f' {tuple(like.shape)}.')
  return value.to(device=like.device, dtype=like.dtype)


def _as_qarray(leaf: Mapping, template: qarray.QArray | None, path, device) -> qarray.QArray:
  qv = torch.as_tensor(leaf['qvalue'])
  qtype = template.qtype if template is not None else (leaf.get('qtype') or numerics.qtype_name(qv.dtype))
  if template is not None:
    qv = _coerce(qv, template.qvalue, path, what='qvalue')
    scale = _coerce(leaf['scale'], template.scale, path, allow_broadcast=True, what='scale')
    zp = leaf.get('zero_point')
    if template.zero_point is None and zp is not None:
      raise ValueError(f'{path} provided an unexpected "zero_point" for a symmetric quantized param.')
    if template.zero_point is not None and zp is None:
      raise ValueError(f'{path} is missing required quantized leaf "zero_point".')
    if zp is not None:
      zp = _coerce(zp, template.zero_point, path, allow_broadcast=True, what='zero_point')
  else:
    qv = qv.to(device)
    scale = torch.as_tensor(leaf['scale']).to(device)
    zp = leaf.get('zero_point')
    zp = None if zp is None else torch.as_tensor(zp).to(device)
  out = qarray.QArray(qv, scale, zp, qtype)
  qarray.validate_qarray(out)
  return out


def process_prequantized_params(checkpoint_params: Mapping[str, Any], template_params: Any, *,
                                allow_extra_params: bool = False) -> dict:
  """checkpoint_util.py:383-501.  `checkpoint_params`: nested dict whose leaves are tensors or
  {'qvalue', 'scale'[, 'zero_point']} dicts.  `template_params`: the PTQ model (or its param
  tree): WithAux(QArray) leaves where the model is quantized, tensors elsewhere.  Returns a tree
  that qwix_b200.model.set_params installs:

    quantized checkpoint, quantized template -> WithAux(QArray) with the template's `how`
    quantized checkpoint, float template     -> the dequantized tensor
    float checkpoint,     float template     -> the tensor, cast to the template's dtype
    float checkpoint,     quantized template -> ValueError
  """
  out = {}
  for path, leaf in _flatten(checkpoint_params):
    resolved, tmpl = _template_at(template_params, path)
    if tmpl is None:
      if not allow_extra_params:
        raise ValueError('Found extra parameters in prequantized_params not present in template:'
                         f' {resolved}')
      logger.info('Skipping parameter not in template: %s', resolved)
      continue
    how = tmpl.how if isinstance(tmpl, ptq.WithAux) else None
    tmpl_array = tmpl.array if isinstance(tmpl, ptq.WithAux) else tmpl
    quantized_tmpl = isinstance(tmpl_array, qarray.QArray)
    if _is_quantized_leaf(leaf) and quantized_tmpl:
      _validate(leaf, resolved)
      qa = _as_qarray(leaf, tmpl_array, resolved, tmpl_array.device)
      processed = ptq.WithAux(qa, how) if how is not None else qa
    elif _is_quantized_leaf(leaf):
      _validate(leaf, resolved)
      qa = _as_qarray(leaf, None, resolved, tmpl_array.device)
      processed = _coerce(qarray.dequantize(qa), tmpl_array, resolved, what='dequantized value')
    elif not quantized_tmpl:
      processed = _coerce(leaf, tmpl_array, resolved, what='value')
    else:
      raise ValueError(f'Unhandled or invalid parameter combination for {resolved}. '
                       f'checkpoint_param is {type(leaf)}, template_param is {type(tmpl)}.')
    out[resolved] = processed
  return _unflatten(out)


def restore_quantization_rules(checkpoint_params: Mapping[str, Any],
                               rule_type=qconfig.QuantizationRule, *, tile_size,
                               act_qtype=_DEFAULT_ACT_QTYPE, **kwargs) -> list:
  """checkpoint_util.py:504-587 -- one rule per module that holds a quantized weight: the module
  path with numeric components turned into wildcards, the weight qtype read off the codes,
  'minmax' when a zero point is present, activations like the weights unless told otherwise."""
  rules = {}
  for path, leaf in _flatten(checkpoint_params):
    if not _is_quantized_leaf(leaf):
      continue
    parts = path[:-1] if path and path[-1] == 'array' else path
    parts = parts[:-1]
    module_path = '/'.join('[^/]+' if isinstance(p, int) or str(p).isdigit() else str(p)
                           for p in parts)
    weight_qtype = leaf.get('qtype') or numerics.qtype_name(torch.as_tensor(leaf['qvalue']).dtype)
    rule = rule_type(
        module_path=module_path, weight_qtype=weight_qtype,
        act_qtype=weight_qtype if act_qtype is _DEFAULT_ACT_QTYPE else act_qtype,
        weight_calibration_method='minmax' if leaf.get('zero_point') is not None else 'absmax',
        tile_size=tile_size, **kwargs)
    if module_path in rules and rules[module_path] != rule:
      logger.warning('Conflicting quantization rules reconstructed for %s. Existing: %s, New: %s.'
                     ' The existing rule will be overwritten.', module_path, rules[module_path], rule)
    rules[module_path] = rule
  return list(rules.values())


# ---- disk ---------------------------------------------------------------------------------------

def _pack_int4(q: torch.Tensor) -> torch.Tensor:
  """[.., C] one code per byte -> [.., C / 2] bytes, low nibble = even index."""
  if q.shape[-1] % 2:
    raise ValueError('int4 codes are packed in pairs along the last axis: its extent must be even.')
  u = (q.to(torch.int16) & 0xf).to(torch.uint8)
  return (u[..., 0::2] | (u[..., 1::2] << 4)).contiguous()


def _unpack_int4(b: torch.Tensor) -> torch.Tensor:
  lo = (b & 0xf).to(torch.int8)
  hi = (b >> 4).to(torch.int8)
  both = torch.stack([lo, hi], dim=-1).reshape(*b.shape[:-1], b.shape[-1] * 2)
  return torch.where(both > 7, both - 16, both).to(torch.int8)


def to_checkpoint_tree(params: Mapping[str, Any]) -> dict:
  """A model's param tree (WithAux / QArray / tensor leaves) as plain checkpoint leaves:
  {'qvalue', 'scale'[, 'zero_point']} dicts and tensors."""
  out = {}
  for path, leaf in _flatten(params):
    arr = leaf.array if isinstance(leaf, ptq.WithAux) else leaf
    if isinstance(arr, qarray.QArray):
      d = {'qvalue': arr.qvalue, 'scale': arr.scale, 'qtype': arr.qtype}
      if arr.zero_point is not None:
        d['zero_point'] = arr.zero_point
      out[path] = d
    else:
      out[path] = arr
  return _unflatten(out)


def save_prequantized(params: Mapping[str, Any], filename: str) -> None:
  """Writes a param tree (as returned by `QuantizedModel.params()` or `quantize_params`) to one
  safetensors file.  Keys are '/'-joined paths plus '.qvalue' / '.scale' / '.zero_point' for
  quantized leaves; qtypes (needed to tell int4 from int8 codes) go to the file's metadata."""
  from safetensors.torch import save_file
  tensors, qtypes = {}, {}
  for path, leaf in _flatten(to_checkpoint_tree(params)):
    key = '/'.join(str(p) for p in path)
    if _is_quantized_leaf(leaf):
      qtype = leaf.get('qtype') or numerics.qtype_name(leaf['qvalue'].dtype)
      qtypes[key] = qtype
      qv = leaf['qvalue']
      tensors[key + '.qvalue'] = _pack_int4(qv) if qtype == 'int4' else qv.contiguous()
      tensors[key + '.scale'] = leaf['scale'].contiguous()
      if leaf.get('zero_point') is not None:
        tensors[key + '.zero_point'] = leaf['zero_point'].contiguous()
    else:
      tensors[key] = leaf.contiguous()
  save_file({k: v.cpu() for k, v in tensors.items()}, filename,
            metadata={'qwix_qtypes': json.dumps(qtypes), 'format': 'qwix_b200.prequantized.v1'})


def load_prequantized(filename: str, device='cpu') -> dict:
  """Reads a file written by save_prequantized back into a checkpoint tree (quantized leaves
  as {'qvalue', 'scale'[, 'zero_point'], 'qtype'} dicts) for process_prequantized_params."""
  from safetensors import safe_open
  flat: dict = {}
  with safe_open(filename, framework='pt', device=str(device)) as f:
    qtypes = json.loads((f.metadata() or {}).get('qwix_qtypes', '{}'))
    for key in f.keys():
      base, _, field = key.rpartition('.')
      if field in _LEAF_NAMES and base in qtypes:
        t = f.get_tensor(key)
        if field == 'qvalue' and qtypes[base] == 'int4':
          t = _unpack_int4(t)
        leaf = flat.setdefault(tuple(base.split('/')), {'qtype': qtypes[base]})
        leaf[field] = t
      else:
        flat[tuple(key.split('/'))] = f.get_tensor(key)
  return _unflatten(flat)
