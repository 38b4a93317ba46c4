"""Import the compiled control plane (page pool, cache manager, scheduler).

The C++ sources under ``csrc/control`` are compiled on first import; see
``einf_b200.ops.build``.
"""
from __future__ import annotations

import importlib.util
import sys

from ..ops import build

_NAME = "einf_b200._control"


def _load():
    module = sys.modules.get(_NAME)
    if module is not None:
        return module
    path = build.build_control_module()
    spec = importlib.util.spec_from_file_location(_NAME, str(path))
    module = importlib.util.module_from_spec(spec)
    sys.modules[_NAME] = module
    spec.loader.exec_module(module)
    return module


_control = _load()

PagePool = _control.PagePool
GroupSpec = _control.GroupSpec
CacheManager = _control.CacheManager
SamplingParams = _control.SamplingParams
RequestSpec = _control.RequestSpec
RequestView = _control.RequestView
ScheduledRequest = _control.ScheduledRequest
BatchPlan = _control.BatchPlan
RequestResult = _control.RequestResult
ExecutionResult = _control.ExecutionResult
Scheduler = _control.Scheduler
SchedulerStats = _control.SchedulerStats
PackConfig = _control.PackConfig
PackedStep = _control.PackedStep
pack_plan = _control.pack_plan
step_buffer_size = _control.step_buffer_size
