"""Contexts for nnabla's test suite under the "b200" extension.

nnabla's function tests take their contexts from a module of this name
(python/test/nbla_test_utils.py:40-46: `from list_context_ext import list`);
putting this file on PYTHONPATH makes `pytest python/test/function/...` of an
nnabla checkout run every function test under cpu:float and under b200:float.
Each entry is (context, function-name suffix); the suffix is what
function_tester appends to the reference name when it checks
Function.name (nbla_test_utils.py:817-818). The extension's classes derive from
the reference classes and keep their names, so the suffix is empty.
"""
import nnabla as nn
from nnabla.ext_utils import get_extension_context

list = [(nn.Context(["cpu:float"], "CpuCachedArray", "0"), ""),
        (get_extension_context("b200", device_id="0"), "")]
