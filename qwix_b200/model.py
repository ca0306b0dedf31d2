"""quantize_model / quantize_params for qwix_b200.nn models.

The reference copies a Flax model and patches its methods so that a provider intercepts
the ops they issue (qwix/_src/model.py:51-151).  Here the wrapper activates the provider
around the model's forward and records, through module hooks, which sub-module is
running -- the '/'-joined path that rules match on (qconfig.py:209-217).
"""

from __future__ import annotations

from typing import Any, Collection

import torch

from qwix_b200 import _context
from qwix_b200 import qconfig
from qwix_b200.providers import ptq


class QuantizedModel(torch.nn.Module):
  """A model whose ops run under a quantization provider."""

  def __init__(self, model: torch.nn.Module, provider: qconfig.QuantizationProvider):
    super().__init__()
    self.model = model
    self.provider = provider
    self._hooks = []
    for name, mod in model.named_modules():
      path = tuple(name.split('.')) if name else ()
      self._hooks.append(mod.register_forward_pre_hook(
          lambda m, args, _p=path: _context.push_module(m, _p)))
      self._hooks.append(mod.register_forward_hook(
          lambda m, args, out: _context.pop_module(), always_call=True))

  def forward(self, *args, _method: str | None = None, **kwargs):
    """Runs the model (or, with `_method`, another method of it that ends in the model's
    ops) under the provider."""
    model, args, kwargs = self.provider.process_model_inputs(self.model, args, kwargs)
    with _context.provider_scope(self.provider):
      out = model(*args, **kwargs) if _method is None else getattr(model, _method)(*args, **kwargs)
    return self.provider.process_model_output(_method or '__call__', out)

  def params(self) -> dict:
    """Nested dict of the model's weights: tensors, or WithAux(QArray) once quantized --
    the tree that quantize_params takes as `abstract_quantized_params`."""
    return get_params(self.model)


def get_params(model: torch.nn.Module) -> dict:
  tree: dict = {}
  for name, mod in model.named_modules():
    node = tree
    if name:
      for part in name.split('.'):
        node = node.setdefault(part, {})
    for pname, p in mod.named_parameters(recurse=False):
      node[pname] = p.data
    for aname, v in vars(mod).items():
      if isinstance(v, ptq.WithAux):
        node[aname] = v
  def prune(d):
    return {k: (prune(v) if isinstance(v, dict) else v) for k, v in d.items()
            if not (isinstance(v, dict) and not prune(v))}
  return prune(tree)


def set_params(model: torch.nn.Module, params: dict):
  """Installs a tree produced by quantize_params (or plain tensors) into the model."""
  def visit(mod, tree):
    for k, v in tree.items():
      if isinstance(v, dict):
        visit(getattr(mod, k), v)
      elif isinstance(v, ptq.WithAux):
        if k in mod._parameters:
          del mod._parameters[k]
        setattr(mod, k, v)
      else:
        if k in mod._parameters:
          mod._parameters[k].data = v
        else:
          if hasattr(mod, k):
            delattr(mod, k)
          mod.register_parameter(k, torch.nn.Parameter(v, requires_grad=False))
  visit(model, params)


def quantize_model(model: torch.nn.Module, provider: qconfig.QuantizationProvider,
                   *model_inputs: Any, methods: Collection[str] = ('__call__',),
                   **model_inputs_kwargs: Any) -> QuantizedModel:
  """model.py:51-89.  With model inputs given (the reference's NNX form) the model is run
  once so that every weight is quantized in place; without them weights are quantized
  the first time their module runs (or offline by quantize_params)."""
  if tuple(methods) != ('__call__',):
    raise ValueError('Only the __call__ method can be quantized on this backend.')
  if isinstance(model, QuantizedModel):
    model = model.model
  q = QuantizedModel(model, provider)
  if model_inputs or model_inputs_kwargs:
    with torch.no_grad():
      q(*model_inputs, **model_inputs_kwargs)
  return q


quantize_params = ptq.quantize_params
