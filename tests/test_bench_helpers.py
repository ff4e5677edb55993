"""Host-side helpers of bench.py that need no GPU."""
import importlib.util
import os


def _bench():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(root, "bench.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_numa_cpus_of_pci_device(tmp_path):
    b = _bench()
    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("16-19,48-49\n")
    assert b.numa_cpus_of_pci_device("0000:1b:00.0", str(tmp_path)) == (1, {16, 17, 18, 19, 48, 49})
    (dev / "numa_node").write_text("-1\n")                       # the machine does not say
    assert b.numa_cpus_of_pci_device("0000:1b:00.0", str(tmp_path)) is None
    assert b.numa_cpus_of_pci_device("0000:ff:00.0", str(tmp_path)) is None     # no such device


def test_reference_arm_prints_unavailable(capsys):
    b = _bench()
    assert b.reference_arm() == 0
    import json
    line = json.loads(capsys.readouterr().out)
    assert line["impl"] == "reference" and "unavailable" in line


def test_check_status_clears_the_words_it_is_given():
    """An error status is raised once; the status word and the barrier / arrival words passed along
    are zero afterwards, so the object that owns them can run again."""
    import pytest
    import torch
    from parameter_server_b200.ops import _lib
    status = torch.tensor([3], dtype=torch.int32)
    sync = torch.tensor([5, 1, 7, 0], dtype=torch.int32)
    with pytest.raises(_lib.PsbCudaError, match="timed out"):
        _lib.check_status(status, "probe", reset=(sync, None))
    assert int(status.item()) == 0 and sync.tolist() == [0, 0, 0, 0]
    _lib.check_status(status, "probe", reset=(sync,))        # clean: no exception
