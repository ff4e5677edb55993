"""mpirun / docker launchers (command construction, no mpirun or docker needed) and the binary
matrix files of the reference's MATLAB helpers."""
import numpy as np
import pytest
import scipy.sparse as sp


def test_mpi_node_roles_and_root_command(tmp_path):
    from parameter_server_b200.system import mpi
    conf = tmp_path / "mpi.conf"
    conf.write_text('num_workers=2\nnum_servers=1\n# comment\nbin="bin/psb_linear"\narg="-app_file x.conf -num_threads 2"\n'
                    'network_interface=eth0\nnetwork_port=8100\nhostfile=hosts.txt\n')
    c = mpi.read_conf(str(conf))
    assert c["arg"] == "-app_file x.conf -num_threads 2" and c["network_port"] == "8100"
    root = mpi.root_command(str(conf), c, "10.0.0.1")
    assert root[:5] == ["mpirun", "-hostfile", "hosts.txt", "-np", "4"] and "role:SCHEDULER,hostname:'10.0.0.1',port:8100,id:'H'" in root
    sched = "role:SCHEDULER,hostname:'10.0.0.1',port:8100,id:'H'"
    roles = []
    for rank in range(4):
        cmd = mpi.node_command(sched, c, rank, 4, "10.0.0.2", 9000 + rank)
        me = cmd[cmd.index("-my_node") + 1]
        roles.append(me.split(",")[0] + "/" + me.split("id:")[1])
        assert cmd[0] == "bin/psb_linear" and cmd[-4:] == ["-app_file", "x.conf", "-num_threads", "2"]
    assert roles == ["role:SCHEDULER/'H'", "role:SERVER/'S0'", "role:WORKER/'W0'", "role:WORKER/'W1'"]
    with pytest.raises(RuntimeError):
        mpi.node_command(sched, c, 0, 3, "10.0.0.2", 9000)
    assert mpi.mpi_rank_and_size({"OMPI_COMM_WORLD_RANK": "3", "OMPI_COMM_WORLD_SIZE": "8"}) == (3, 8)
    assert mpi.mpi_rank_and_size({"PMI_RANK": "1", "PMI_SIZE": "2"}) == (1, 2)
    with pytest.raises(RuntimeError):
        mpi.mpi_rank_and_size({})


def test_docker_local_commands(tmp_path, capsys):
    from parameter_server_b200.system import docker
    cmds = docker.local_commands(1, 2, "app.conf", "data", "model", ["-num_threads", "2"], "172.17.0.1")
    assert len(cmds) == 4 and all(c[:3] == ["docker", "run", "--rm"] for c in cmds)
    names = [c[c.index("--name") + 1] for c in cmds]
    assert names == ["n0", "n1", "n2", "n3"]
    nodes = [c[c.index("-my_node") + 1] for c in cmds]
    assert "SCHEDULER" in nodes[0] and "id:'S0'" in nodes[1] and "id:'W1'" in nodes[3] and "port:8003" in nodes[3]
    assert all(c[c.index("-scheduler") + 1] == nodes[0] for c in cmds)
    assert docker.main(["--dry-run", "rm", "1", "2"]) == 0
    assert capsys.readouterr().out.strip() == "docker rm -f n0 n1 n2 n3"


def test_root_node_string_and_s3_upload_command(tmp_path, capsys):
    """`launch root-node IFACE PORT` prints the -scheduler string of this machine; `docker upload` is one curl
    call with the object's size and a public-read ACL."""
    from parameter_server_b200.system import docker, launch
    assert launch.main(["root-node", "lo", "8000"]) == 0
    assert capsys.readouterr().out.strip() == "role:SCHEDULER,hostname:'127.0.0.1',port:8000,id:'H'"
    f = tmp_path / "app.conf"
    f.write_text("x" * 37)
    assert docker.main(["--dry-run", "upload", str(f), "s3://mybucket/jobs/app.conf"]) == 0
    out = capsys.readouterr().out.strip()
    assert out == f"curl 'http://mybucket.s3.amazonaws.com/jobs/app.conf?Content-Length=37&x-amz-acl=public-read' --upload-file {f}"
    with pytest.raises(SystemExit):
        docker.main(["--dry-run", "upload", str(f), "/not/s3"])


def test_binary_matrix_files_round_trip(tmp_path):
    from parameter_server_b200.utils import binfmt
    rng = np.random.default_rng(0)
    X = sp.random(40, 30, density=0.2, random_state=1, format="csr")
    y = np.where(rng.random(40) < 0.5, 1.0, -1.0)
    binfmt.mat2bin(str(tmp_path / "m"), y, X)
    X2, y2 = binfmt.bin2mat(str(tmp_path / "m"))
    assert (abs(X - X2) > 1e-12).nnz == 0 and np.array_equal(y, y2)
    Xb = (X > 0).astype(float)
    binfmt.mat2bin(str(tmp_path / "b"), y, Xb)
    assert not (tmp_path / "b.value").exists()
    Xb2, _ = binfmt.bin2mat(str(tmp_path / "b"))
    assert (Xb != Xb2).nnz == 0
    assert np.array_equal(binfmt.load_bin(str(tmp_path / "m.label"), "float64", offset=3, length=4), y[3:7])
    Xf, go = binfmt.filter_fea(Xb, [0, 10, 30], min_count=4)
    counts = np.asarray(Xb.sum(axis=0)).ravel()
    assert Xf.shape[1] == int((counts > 4).sum()) and go[0] == 0 and go[-1] == Xf.shape[1]
    assert go[1] == int((counts[:10] > 4).sum())
    # the text writer produces what the PS text parser reads
    from parameter_server_b200.system import core
    binfmt.saveas_pserver(str(tmp_path / "t.txt"), y, X, group_id=np.repeat([0, 1], 15))
    first = open(tmp_path / "t.txt").readline()
    ex = core.parse_example(first, "SPARSE")
    got = np.concatenate([ex[g]["key"] for g in sorted(k for k in ex if isinstance(k, int))]) if ex else []
    assert sorted(int(k) for k in got) == sorted(X[0].indices.tolist())


def test_bin_reader_and_writer(tmp_path, capsys):
    """Minibatches from mapped binary matrices: the reference's MATLAB layout (32-bit ids, float64 values) and
    the converter's (64-bit ids, float32 values); rows, offsets and values match the matrix; a minibatch stays
    valid while the next one is read."""
    from parameter_server_b200.utils import binfmt, datatool
    rng = np.random.default_rng(0)
    X = sp.random(300, 5000, density=0.01, random_state=1, format="csr", dtype=np.float64)
    X.data = np.round(X.data * 8 + 1) / 4
    y = np.where(rng.random(300) < 0.5, 1.0, -1.0)
    binfmt.mat2bin(str(tmp_path / "a"), y, X)
    r = binfmt.BinReader([str(tmp_path / "a.index"), str(tmp_path / "a.offset"), str(tmp_path / "a.info")])
    assert r.names == [str(tmp_path / "a")]
    first = r.read_matrices(128)
    second = r.read_matrices(128)
    Xs = X.copy(); Xs.sort_indices()
    for k, (yy, (m,)) in enumerate([first, second]):        # `first` was not overwritten by reading `second`
        r0, r1 = k * 128, (k + 1) * 128
        assert np.array_equal(yy, y[r0:r1].astype(np.float32))
        assert np.array_equal(m["offset"], (Xs.indptr[r0:r1 + 1] - Xs.indptr[r0]).astype(np.uint64))
        assert np.array_equal(m["index"], Xs.indices[Xs.indptr[r0]:Xs.indptr[r1]].astype(np.uint64))
        assert np.allclose(m["value"], Xs.data[Xs.indptr[r0]:Xs.indptr[r1]]) and not m["binary"]
    third = r.read_matrices(128)
    assert len(third[0]) == 300 - 256 and r.read_matrices(128) is None
    # text -> binary matrix with 64-bit ids, and back
    big = (1 << 40) + 5
    (tmp_path / "part-0").write_text(f"1 3:1 {big}:1\n-1 2:1\n")
    (tmp_path / "part-1").write_text("1 9:1\n")
    assert datatool.main(["convert", "-input", str(tmp_path / "part-.*"), "-output", str(tmp_path / "all"), "-to", "bin"]) == 0
    assert "3 examples, 4 nonzeros" in capsys.readouterr().out
    yy, (m,) = binfmt.BinReader([str(tmp_path / "all")]).read_matrices(10)
    assert list(yy) == [1, -1, 1] and list(m["index"]) == [3, big, 2, 9] and list(m["offset"]) == [0, 2, 3, 4]
    # the C++ stream reader (what the CPU nodes use) reads both layouts row by row
    from parameter_server_b200.system import core
    y2, mats = core.StreamReader([str(tmp_path / "all")], "BIN", "LIBSVM", True).read_matrices(10)
    assert list(y2) == [1, -1, 1] and list(mats[0]["index"]) == [3, big, 2, 9] and list(mats[0]["offset"]) == [0, 2, 3, 4]
    assert core.search_files([str(tmp_path / "a.*")], None, "BIN") == [str(tmp_path / "a"), str(tmp_path / "all")]
    rd = core.StreamReader([str(tmp_path / "a")], "BIN", "LIBSVM", True)
    y3, mats = rd.read_matrices(200)
    assert np.array_equal(y3, y[:200].astype(np.float32))
    assert np.array_equal(mats[0]["index"], Xs.indices[:Xs.indptr[200]].astype(np.uint64))
    assert np.allclose(mats[0]["value"], Xs.data[:Xs.indptr[200]])
    y4, _ = rd.read_matrices(200)
    assert len(y4) == 100 and rd.read_matrices(200) is None
