"""Call plans: a graph's forward pass recorded once as the list of library calls it makes, replayed
without the Python operator classes, and optionally captured into one CUDA graph.

The reference's interpreter (nn/__init__.py:408-456) walks its node list on every run and each node
marshals its operands again (nn/__init__.py:189-344).  For a graph whose shapes do not change that
work is the same every time, and at eight ranks per host it is what the GPUs end up waiting for.
``Graph.plan`` therefore runs the forward pass once through a recording stand-in for the library:

* every operator call (``*_forward``) is kept as ``(function, arguments)`` with the very ctypes
  objects the operator class built -- tensor handles, attribute structs, scalars;
* every tensor that appears in a recorded call gets one more reference, so outputs, scratch views
  and intermediate edges stay alive (and at the same addresses) for as long as the plan exists;
* allocation, release, reference counting and transfers are passed through and not recorded.

``GraphPlan.run`` replays the list: one ctypes call per recorded operator call, nothing else.
``GraphPlan.capture`` replays it once more inside ``tops_capture_begin`` / ``tops_capture_end``; from
then on ``run`` is a single ``tops_capture_launch``.  Inputs are copied (device to device) into buffers the
plan owns; outputs are the tensors of the recording pass, overwritten by every run.  A plan is valid for the input shapes and dtypes it was recorded with, and
for graphs whose control flow does not depend on tensor contents (a node that reads a tensor back
to the host while recording is refused).
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence

from .. import capi
from ..capi import CQConvCall, TensorP

# struct members of QConvCall that hold tensor handles
_QCONV_TENSOR_FIELDS = ("x", "x_scale", "x_zero", "w_codes", "w_scale", "bias", "residual", "y", "y_levels", "next_scale", "next_zero")
# calls that are part of the computation although their names do not end in _forward
_ALSO_RECORDED = {"tops_dynamic_quantize_range", "tops_dynamic_quantize_apply"}
# calls that move data to the host or wait for the device: a forward pass that needs them cannot be replayed blindly
_REFUSED = {"tops_download", "tops_download_async", "tops_sync"}


class _Recorder:
    """Stands in for the ctypes library object while a forward pass is recorded."""

    def __init__(self, lib):
        self._lib = lib
        self.calls: List[tuple] = []
        self.held: List[object] = []          # tensor handles this recording holds a reference to
        self.recording = True                 # afterwards every call passes straight through (tensors made while
                                              # recording keep this object as their library handle)

    def _hold(self, handle) -> None:
        if handle:
            self._lib.tops_retain(handle)
            self.held.append(handle)

    def _hold_arguments(self, name, args) -> None:
        for a in args:
            if isinstance(a, TensorP):
                self._hold(a)
            elif name == "tops_qconv_forward" and isinstance(getattr(a, "_obj", None), CQConvCall):
                call = a._obj
                for field in _QCONV_TENSOR_FIELDS:
                    ptr = getattr(call, field)
                    if ptr:
                        self._hold(ctypes.cast(ptr, TensorP))

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if not self.recording:
            return fn
        if name in _REFUSED:
            def refused(*args):
                raise capi.TensorOpsError(f"{name} was called while a call plan was being recorded: this graph reads tensors "
                                          "on the host during its forward pass and cannot be replayed")
            return refused
        if not (name.endswith("_forward") or name in _ALSO_RECORDED):
            return fn

        def recorded(*args):
            self._hold_arguments(name, args)
            self.calls.append((fn, args))
            return fn(*args)
        return recorded

    def release(self) -> None:
        held, self.held = self.held, []
        for handle in held:
            self._lib.free_tensor(handle)


class GraphPlan:
    """The recorded forward pass of one ``Graph`` for fixed input shapes (see the module docstring)."""

    def __init__(self, graph, inputs: Sequence[object]):
        from . import Ops
        self.graph = graph                    # keeps nodes, attribute arrays and initializers alive
        self.lib = Ops._get_lib()
        graph.make_resident()
        # the plan's own input buffers (copies of the example inputs): a caller's tensor is never aliased, so a later
        # run(other) cannot overwrite it
        from . import Tensor
        from ..device import DeviceArray
        self.inputs = []
        for t in inputs:
            src = t.to_device()
            mine = DeviceArray.empty(tuple(src.data.shape), src.dtype, lib=self.lib)
            self.lib.flatten_forward(src.data.handle, mine.handle)
            self.inputs.append(Tensor(*src.size, dtype=src.dtype, data=mine))
        self._captured = None
        recorder = _Recorder(self.lib)
        Ops._recorder = recorder
        try:
            outs = graph.forward(*self.inputs)
        finally:
            Ops._recorder = None
            recorder.recording = False
        capi.check(self.lib)
        self._recorder = recorder
        self.outputs = outs
        self.calls = recorder.calls

    # -- running -----------------------------------------------------------------------------------
    def _feed(self, inputs) -> None:
        if len(inputs) != len(self.inputs):
            raise ValueError(f"plan takes {len(self.inputs)} inputs, got {len(inputs)}")
        for mine, given in zip(self.inputs, inputs):
            if given is mine or given.data is mine.data:
                continue                      # the caller wrote into the plan's own buffer
            src = given.to_device()
            if tuple(src.data.shape) != tuple(mine.data.shape) or src.dtype != mine.dtype:
                raise ValueError(f"plan was recorded for input {tuple(mine.data.shape)} {mine.dtype}, got {tuple(src.data.shape)} {src.dtype}")
            self.lib.flatten_forward(src.data.handle, mine.data.handle)      # device-to-device copy on the same stream

    def run(self, *inputs):
        """One forward pass.  Without arguments the plan's own input tensors are used as they are (write
        into ``plan.inputs[i]`` beforehand); otherwise the given tensors are copied into them first.
        Returns the output tensor(s) of the recording pass, overwritten in place."""
        if inputs:
            self._feed(inputs)
        if self._captured:
            if self.lib.tops_capture_launch(self._captured):
                capi.check(self.lib)
        else:
            for fn, args in self.calls:
                fn(*args)
        return self.outputs

    def capture(self) -> bool:
        """Turn the recorded list into one CUDA graph.  Returns False (and keeps replaying call by call)
        when the driver cannot capture the sequence."""
        if self._captured:
            return True
        if self.lib.tops_capture_begin():
            self.lib.tops_clear_error()
            return False
        for fn, args in self.calls:
            fn(*args)
        handle = self.lib.tops_capture_end()
        if not handle or self.lib.tops_last_error():
            self.lib.tops_clear_error()
            if handle:
                self.lib.tops_capture_free(handle)
            return False
        self._captured = handle
        return True

    @property
    def captured(self) -> bool:
        return bool(self._captured)

    def close(self) -> None:
        if self._captured:
            self.lib.tops_capture_free(self._captured)
            self._captured = None
        self.calls = []
        if self._recorder is not None:
            self._recorder.release()
            self._recorder = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
