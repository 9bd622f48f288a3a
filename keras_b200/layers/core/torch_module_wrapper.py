"""``TorchModuleWrapper``: use any ``torch.nn.Module`` as a layer; its parameters become tracked variables
(keras/src/utils/torch_utils.py:15-170)."""

import base64
import io

import torch

from keras_b200 import tree
from keras_b200.core.export_registry import keras_export
from keras_b200.core.tensor import get_device
from keras_b200.core.variables import Variable
from keras_b200.layers.layer import Layer
from keras_b200.saving.serialization_lib import in_safe_mode


@keras_export("keras.layers.TorchModuleWrapper")
class TorchModuleWrapper(Layer):
    def __init__(self, module, name=None, output_shape=None, **kwargs):
        super().__init__(name=name, **kwargs)
        object.__setattr__(self, "module", module.to(get_device()))
        self.output_shape = output_shape
        self._track_module_parameters()

    def _has_lazy(self):
        return any(isinstance(p, torch.nn.parameter.UninitializedParameter) for p in self.module.parameters())

    def _track_module_parameters(self):
        if self._has_lazy():
            return
        self._tracker_unlock() if hasattr(self, "_tracker_unlock") else None
        for p in self.module.parameters():
            v = Variable(initializer=p, trainable=p.requires_grad, name="torch_param")
            if p.requires_grad:
                self._trainable_variables.append(v)
            else:
                self._non_trainable_variables.append(v)
        self._invalidate() if hasattr(self, "_invalidate") else None
        self.built = True

    def parameters(self, recurse=True):
        return self.module.parameters(recurse=recurse)

    def build(self, input_shape=None):
        if not self.built:
            if self._has_lazy() and input_shape is not None:
                sample = tree.map_shape_structure(lambda s: torch.zeros([1 if d is None else d for d in s], device=get_device()), input_shape)
                with torch.no_grad():
                    self.module(sample) if not isinstance(sample, (list, tuple)) else self.module(*sample)
            self._track_module_parameters()

    def call(self, *args, training=None, **kwargs):
        if training is False:
            self.module.eval()
        else:
            self.module.train()
        return self.module(*args, **kwargs)

    def save_own_variables(self, store):
        state = self.module.state_dict()
        for key in state.keys():
            store[key] = state[key].detach().cpu().numpy()

    def load_own_variables(self, store):
        state = {}
        for key in store.keys():
            if isinstance(key, bytes):
                key = key.decode()
            state[key] = torch.as_tensor(store[key])
        self.module.load_state_dict(state)

    def compute_output_shape(self, input_shape):
        if self.output_shape is not None:
            return self.output_shape
        # run the module once on zeros (unknown dimensions become 1) and read the result's shape
        sample = tree.map_shape_structure(lambda s: torch.zeros([1 if d is None else d for d in s], device=get_device()), input_shape)
        was_training = self.module.training
        self.module.eval()
        try:
            with torch.no_grad():
                out = self.module(sample) if not isinstance(sample, (list, tuple)) else self.module(*sample)
        finally:
            self.module.train(was_training)
        batch = input_shape[0] if isinstance(input_shape, tuple) and input_shape and not isinstance(input_shape[0], (tuple, list)) else None
        return tree.map_structure(lambda t: (batch,) + tuple(t.shape[1:]), out)

    def get_config(self):
        buffer = io.BytesIO()
        torch.save(self.module, buffer)
        return {**super().get_config(), "module": base64.b64encode(buffer.getvalue()).decode("ascii"), "output_shape": self.output_shape}

    @classmethod
    def from_config(cls, config):
        if "module" in config:
            if in_safe_mode():
                raise ValueError("Requested the deserialization of a `torch.nn.Module` object via `torch.load()`. This carries a potential risk of "
                                 "arbitrary code execution and thus it is disallowed by default. If you trust the source of the artifact, you can "
                                 "override this error by passing `safe_mode=False` to the loading function, or calling "
                                 "`keras.config.enable_unsafe_deserialization().")
            data = config["module"]
            buffer = io.BytesIO(base64.b64decode(data) if isinstance(data, str) else data)
            config["module"] = torch.load(buffer, weights_only=False)
        return cls(**config)
