"""``DcgmContextManager`` against fake DCGM bindings: the sampling thread records the watched fields of this rank's GPU,
and without bindings the optional form is a no-op.  (Nothing here talks to a GPU or changes a setting.)"""

import sys
import time
import types

import pytest


def _install_fake(monkeypatch, tmp_path):
    calls = {"watch": 0, "unwatch": 0, "added": []}

    class _Val:
        def __init__(self, v):
            self.value = v

    class _Samples:
        def WatchFields(self, fields, interval_us, max_age, max_samples):
            calls["watch"] += 1

        def UnwatchFields(self, fields):
            calls["unwatch"] += 1

        def GetLatest(self, fields):
            ids = fields.fieldIds
            return types.SimpleNamespace(values={0: {fid: [_Val(float(fid) / 10.0)] for fid in ids}})

    class DcgmHandle:
        def __init__(self, ipAddress=None, opMode=None):
            self.ip = ipAddress

    class DcgmGroup:
        def __init__(self, handle, groupName=None, groupType=None):
            self.samples = _Samples()

        def AddGpu(self, gpu):
            calls["added"].append(gpu)

    class DcgmFieldGroup:
        def __init__(self, handle, name=None, fieldIds=None):
            self.fieldIds = list(fieldIds)

    pyd = types.ModuleType("pydcgm")
    pyd.DcgmHandle, pyd.DcgmGroup, pyd.DcgmFieldGroup = DcgmHandle, DcgmGroup, DcgmFieldGroup
    structs = types.ModuleType("dcgm_structs")
    structs.DCGM_OPERATION_MODE_AUTO, structs.DCGM_GROUP_EMPTY = 1, 2
    monkeypatch.setitem(sys.modules, "pydcgm", pyd)
    monkeypatch.setitem(sys.modules, "dcgm_fields", types.ModuleType("dcgm_fields"))
    monkeypatch.setitem(sys.modules, "dcgm_structs", structs)
    return calls


def test_samples_with_fake_bindings(monkeypatch, tmp_path):
    from cornstarch_b200.testing.dcgm import FIELDS, DcgmContextManager

    calls = _install_fake(monkeypatch, tmp_path)
    monkeypatch.setenv("LOCAL_RANK", "0")
    dcgm = DcgmContextManager(bindings=str(tmp_path), interval_us=1000)
    assert dcgm.available and calls["added"] == [0]
    with dcgm.profile():
        time.sleep(0.05)
    assert calls["watch"] == 1 and calls["unwatch"] == 1
    trace = dcgm.get_tensor_core_util_trace()
    assert len(trace) >= 5 and all(v == FIELDS["tensor_active"] / 10.0 for _, v in trace)
    assert len(dcgm.get_sm_occupancy_trace()) == len(dcgm.get_sm_active_trace()) == len(dcgm.get_memory_usage_trace()) == len(trace)


def test_optional_without_bindings(tmp_path):
    from cornstarch_b200.testing.dcgm import DcgmContextManager

    for name in ("pydcgm", "dcgm_fields", "dcgm_structs"):
        sys.modules.pop(name, None)
    with pytest.raises(RuntimeError):
        DcgmContextManager(bindings=str(tmp_path))
    dcgm = DcgmContextManager(bindings=str(tmp_path), optional=True)
    assert not dcgm.available
    with dcgm.profile():
        pass
    assert dcgm.get_sm_active_trace() == []
