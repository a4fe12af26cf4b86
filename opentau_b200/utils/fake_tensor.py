"""``FakeTensorContext``: build and step a model on meta-like fake tensors to validate shapes and graph wiring
without allocating weights (reference ``src/opentau/utils/fake_tensor.py:41-81``)."""

from __future__ import annotations

from contextlib import ContextDecorator

from torch._subclasses.fake_tensor import FakeTensorMode


class FakeTensorContext(ContextDecorator):
    _mode = None

    def __init__(self, allow_non_fake_inputs: bool = True):
        self.allow = allow_non_fake_inputs

    def __enter__(self):
        if FakeTensorContext._mode is None:
            FakeTensorContext._mode = FakeTensorMode(allow_non_fake_inputs=self.allow)
        self.mode = FakeTensorContext._mode
        self.mode.__enter__()
        return self

    def __exit__(self, *exc):
        self.mode.__exit__(*exc)
        return False
