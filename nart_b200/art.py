"""The Python runtime interface of the reference (``nart.art``: python/nart/art/__init__.py:15-73 and the
pybind classes of python/src/art/module.cpp:285-526 of ModelTC/NART) on top of the GPU case runner:

    ctx = create_context_from_json("engine.bin.json")     # {"workspaces": {"b200": {}}, "input_workspace": "b200"}
    parade = load_parade("engine.bin", ctx)
    inputs, outputs = get_empty_io(parade)
    inputs[name][:] = data
    parade.run(inputs, outputs)

Same names, arguments, return values and errors: ``run`` checks that every input and output is given
with the parade's shape and dtype (ValueError "input shape not match" and the like), copies the inputs
in, runs, copies the outputs out and returns True; ``reshape`` takes ``{input name: [n, c, h, w]}``,
rebuilds the case for the new shape and returns True.  One backend exists here, so a context must
name the workspace "b200" and nothing else.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np

from . import engine

_DTYPE_NAME = {engine.DT_UINT8: "uint8", engine.DT_INT8: "int8", engine.DT_FLOAT32: "float32", engine.DT_INT32: "int32"}


class RuntimeContext:
    """The workspaces a parade may place its ops on (module.cpp:510-524).  Only "b200" can be loaded."""

    def __init__(self, modules: List[str], input_module: str):
        modules = list(modules)
        for m in modules:
            if m != "b200":
                raise RuntimeError("module [%s] not found: this runtime serves the workspace \"b200\" only" % m)
        if not modules:
            raise RuntimeError("a context needs at least one workspace")
        if input_module != "b200":
            raise RuntimeError("input workspace [%s] is not among the loaded workspaces" % input_module)
        self._modules = modules
        self.input_module = input_module

    @property
    def loaded_workspaces(self) -> List[str]:
        return list(self._modules)


def create_context_from_json(json_path: str) -> RuntimeContext:
    import json
    with open(json_path, "r") as fp:
        ws_data = json.loads(fp.read())
    return RuntimeContext(list(ws_data["workspaces"].keys()), ws_data["input_workspace"])


def create_context_for_target(target: str) -> RuntimeContext:
    if target != "b200":
        raise KeyError(target)
    return RuntimeContext(["b200"], "b200")


class Parade:
    """A loaded case.  ``buf`` is the content of a version-2 engine.bin."""

    def __init__(self, buf: bytes, context: RuntimeContext):
        import os
        import tempfile
        if not isinstance(context, RuntimeContext):
            raise TypeError("Parade needs a RuntimeContext")
        fd, path = tempfile.mkstemp(suffix=".bin")
        try:
            with os.fdopen(fd, "wb") as f:
                f.write(bytes(buf))
            self._model = engine.read_engine(path)
        finally:
            os.unlink(path)
        self._inp = self._model["inputs"][0]
        self._case = None
        self._build(tuple(int(d) for d in self._inp["dims"]))

    # -- construction ---------------------------------------------------------------------------
    def _build(self, nchw):
        import torch
        if self._case is not None:
            self._case.close()
            self._case = None
        n, chw = int(nchw[0]), tuple(int(d) for d in nchw[1:])
        self._case, outs = engine.engine_to_case(self._model, n, input_chw=chw)
        self._batch = n
        self._in_shape = (n,) + chw
        self._out_spec = [((np.float32 if is_f32 else np.uint8), tuple(int(d) for d in shape)) for is_f32, shape in outs]
        self._stream = torch.cuda.Stream()

    def close(self):
        if self._case is not None:
            self._case.close()
            self._case = None

    # -- introspection (module.cpp:302-379, 479-509) ---------------------------------------------
    def get_input_names(self) -> List[str]:
        return [self._inp["name"]]

    def get_output_names(self) -> List[str]:
        return [o["name"] for o in self._model["outputs"]]

    def input_shapes(self) -> Dict[str, List[int]]:
        return {self._inp["name"]: list(self._in_shape)}

    def output_shapes(self) -> Dict[str, List[int]]:
        return {o["name"]: [self._batch] + list(shape) for o, (_, shape) in zip(self._model["outputs"], self._out_spec)}

    def input_dtypes(self) -> Dict[str, str]:
        return {self._inp["name"]: _DTYPE_NAME[self._inp["dtype"]]}

    def output_dtypes(self) -> Dict[str, str]:
        return {o["name"]: np.dtype(dt).name for o, (dt, _) in zip(self._model["outputs"], self._out_spec)}

    def get_tensor_shape(self, name: str) -> List[int]:
        shapes = dict(self.input_shapes(), **self.output_shapes())
        if name not in shapes:
            raise KeyError("tensor %r is neither an input nor an output of the parade" % name)
        return shapes[name]

    def get_tensor_dtype(self, name: str) -> str:
        dtypes = dict(self.input_dtypes(), **self.output_dtypes())
        if name not in dtypes:
            raise KeyError("tensor %r is neither an input nor an output of the parade" % name)
        return dtypes[name]

    # -- running ----------------------------------------------------------------------------------
    def reshape(self, shapes: Dict[str, List[int]]) -> bool:
        """{input name: [n, c, h, w]} -> the case is rebuilt and prepared for that shape (the reference:
        parade_apply_reshape followed by prepare).  False when a name is not an input."""
        for name, dims in shapes.items():
            if name != self._inp["name"] or len(dims) != 4:
                return False
        for dims in shapes.values():
            self._build(tuple(int(d) for d in dims))
        return True

    def forward(self) -> None:
        """Runs on the tensors as they are on the device."""
        self._case.run_device(self._batch, self._stream.cuda_stream)
        self._stream.synchronize()

    def run(self, inputs: dict, outputs: dict) -> bool:
        name = self._inp["name"]
        if name not in inputs:
            raise ValueError("some input not given when calling parade.run")
        x = np.asarray(inputs[name])
        if x.ndim != len(self._in_shape):
            raise ValueError("input dim size not match")
        if tuple(x.shape) != self._in_shape:
            raise ValueError("input shape not match")
        if x.dtype.name != _DTYPE_NAME[self._inp["dtype"]]:
            raise ValueError("input dtype not match")
        want_shapes, want_dtypes = self.output_shapes(), self.output_dtypes()
        for oname in self.get_output_names():
            if oname not in outputs:
                raise ValueError("some output not given when calling parade.run")
            y = outputs[oname]
            if y.ndim != len(want_shapes[oname]):
                raise ValueError("output dim size not match")
            if list(y.shape) != want_shapes[oname]:
                raise ValueError("output shape not match")
            if y.dtype.name != want_dtypes[oname]:
                raise ValueError("output dtype not match")
        results = self._case.run_host([np.ascontiguousarray(x)], self._out_spec, self._stream.cuda_stream)
        for oname, arr in zip(self.get_output_names(), results):
            outputs[oname][...] = arr.reshape(outputs[oname].shape)
        return True


def load_parade(engine_fp: str, ctx: RuntimeContext) -> Parade:
    with open(engine_fp, "rb") as fp:
        return Parade(fp.read(), ctx)


def get_empty_io(parade: Parade) -> Tuple[dict, dict]:
    inputs = {k: np.zeros(v, dtype=np.dtype(parade.get_tensor_dtype(k))) for k, v in parade.input_shapes().items()}
    outputs = {k: np.zeros(v, dtype=np.dtype(parade.get_tensor_dtype(k))) for k, v in parade.output_shapes().items()}
    return inputs, outputs
