"""The host-runtime throughput probes (counterparts of network_perf_ps / kv_map_perf_ps /
kv_layer_perf_ps) run end to end over in-process nodes and report sane numbers."""
from parameter_server_b200.system import perf


def test_network_probe():
    r = perf.main(["network", "--data-size", "64", "--n", "10"])
    assert r["MB_per_s_per_worker"] > 1 and r["messages"] == 10


def test_kv_map_probe_pull_depends_on_push():
    r = perf.main(["kv_map", "--keys", "5000", "--n", "2"])
    assert 0 < r["keys"] <= 5000 and r["keys_per_s_per_worker"] > 1000


def test_kv_layer_probe():
    r = perf.main(["kv_layer", "--n", "1", "-ns", "2", "-nw", "1"])
    assert r["MB_per_s_per_worker"] > 1 and len(r["layer_elements"]) == 7
