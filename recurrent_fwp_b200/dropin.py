"""Put this package's kernels under the module names the reference's layer code imports.

The reference's three sub-projects import the fast-weight ops by module name:

  algorithmic/layers.py:7-10
      ``from fast_weight import fast_weight_delta`` (script directory on ``sys.path``)
  language_modeling/src/utils/cuda_fast_weight_layer.py:9-23
      ``from utils.fast_fast_weight import fast_weight_delta``, ``utils.fast_weight_rnn``, ``utils.fast_lstm*`` ...
  reinforcement_learning/torchbeast/layer.py:7-10
      ``from torchbeast.fast_weight import fast_weight_delta`` ...

``activate`` makes those imports resolve to the sub-packages of ``recurrent_fwp_b200`` while every other module of
the reference (``utils.performer_helper``, ``torchbeast.core`` ...) still comes from the reference checkout, which
is neither edited nor copied.  Call it once, before the reference's layer file is imported:

    from recurrent_fwp_b200 import dropin
    dropin.activate('language_modeling', '/path/to/recurrent-fwp')
    from utils.cuda_fast_weight_layer import CudaFastWeightLinearTransformerLayer
"""
import importlib
import os
import sys
import types

_PKG = os.path.dirname(os.path.abspath(__file__))

# sub-project -> (directory to put on sys.path, package the kernels are sub-modules of, its directory)
_LAYOUT = {
    'algorithmic': ('algorithmic', None, None),
    'language_modeling': (os.path.join('language_modeling', 'src'), 'utils', os.path.join('language_modeling', 'src', 'utils')),
    'reinforcement_learning': ('reinforcement_learning', 'torchbeast', os.path.join('reinforcement_learning', 'torchbeast')),
}
KERNEL_MODULES = ('fast_weight', 'fast_transformers', 'rec_update_fwm_tanh', 'fast_weight_rnn_v2', 'fast_weight_rnn',
                  'fast_lstm', 'fast_lstm_v2', 'fast_lstm_v3', 'fast_lstm_v4')
# the language-model code calls the delta rule ``fast_fast_weight``
_ALIASES = {'fast_fast_weight': 'fast_weight'}


def activate(project, reference_root):
    """Make ``project``'s layer code import this package's ops.  ``project`` is 'algorithmic', 'language_modeling'
    or 'reinforcement_learning'; ``reference_root`` is the root of a recurrent-fwp checkout."""
    if project not in _LAYOUT:
        raise ValueError('unknown sub-project %r (one of %s)' % (project, ', '.join(sorted(_LAYOUT))))
    script_dir, parent, parent_dir = _LAYOUT[project]
    script_dir = os.path.join(reference_root, script_dir)
    if not os.path.isdir(script_dir):
        raise FileNotFoundError('%s is not a recurrent-fwp checkout (no %s)' % (reference_root, script_dir))
    ours = {name: importlib.import_module('recurrent_fwp_b200.' + name) for name in KERNEL_MODULES}
    if parent is None:
        # the kernels are top-level modules found through the script directory: register ours under those names
        for name, mod in ours.items():
            sys.modules[name] = mod
    else:
        # the kernels are sub-modules of the reference's own package: an overlay package whose search path lists
        # this package first and the reference's directory second
        pkg = types.ModuleType(parent)
        pkg.__path__ = [_PKG, os.path.join(reference_root, parent_dir)]
        pkg.__package__ = parent
        sys.modules[parent] = pkg
        for name, mod in ours.items():
            sys.modules[parent + '.' + name] = mod
            setattr(pkg, name, mod)
        for alias, name in _ALIASES.items():
            sys.modules[parent + '.' + alias] = ours[name]
            setattr(pkg, alias, ours[name])
    if script_dir not in sys.path:
        sys.path.append(script_dir)
    return ours
