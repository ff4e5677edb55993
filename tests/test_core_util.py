"""Host utilities, filters, parsers and data readers of the C++ runtime."""
import gzip
import os

import numpy as np
import pytest

from parameter_server_b200.system import core


# ---------------------------------------------------------------- hashes / sketches
def test_crc32c_and_murmur_known_vectors():
    assert core.crc32c(b"123456789") == 0xE3069283          # standard CRC-32C check value
    assert core.crc32c(b"") == 0
    assert core.crc32c_extend(core.crc32c(b"1234"), b"56789") == 0xE3069283
    assert core.crc32c_unmask(core.crc32c_mask(0xDEADBEEF)) == 0xDEADBEEF
    assert core.murmurhash3_x86_32(b"", 0) == 0
    assert core.murmurhash3_x86_32(b"hello", 0) == 0x248BFA47
    assert core.murmurhash3_x86_32(b"hello, world", 0) == 0x149BBB7F
    assert core.murmurhash3_x64_128(b"", 0) == (0, 0)
    assert core.murmurhash3_x64_128(b"hello", 0) == (0xCBD8A7B341BD9B02, 0x5B1E906A48AE1D19)
    # every tail length of the three variants (0..49 bytes, three seeds), against a digest taken from an
    # implementation that had been checked against the published vectors above
    import hashlib
    data = bytes((i * 37 + 11) % 256 for i in range(80))
    h = hashlib.sha256()
    for n in range(50):
        for seed in (0, 1, 512927377):
            h.update(repr((core.murmurhash3_x86_32(data[:n], seed), core.murmurhash3_x86_128(data[:n], seed),
                           core.murmurhash3_x64_128(data[:n], seed))).encode())
    assert h.hexdigest() == "7675e6d440d3154dc82809d766e11cf38f3cf6a8e114f448534946f3f1745231"
    a, b = core.murmurhash3_x64_128(b"abcdefghijklmnopqrstuvwxyz", 512927377)
    assert (a, b) != core.murmurhash3_x64_128(b"abcdefghijklmnopqrstuvwxyy", 512927377)


def test_countmin_bloom_bitmap():
    rng = np.random.default_rng(0)
    keys = np.unique(rng.integers(0, 1 << 62, 3000, dtype=np.uint64))
    cm = core.CountMin(); cm.resize(1 << 15, 2, 255)
    cnt = rng.integers(1, 40, len(keys)).astype(np.uint8)
    cm.insert_many(keys, cnt)
    q = cm.query_many(keys)
    assert (q >= cnt).all() and (q == cnt).mean() > 0.8          # over-estimates only
    cm.insert(int(keys[0]), 250); cm.insert(int(keys[0]), 250)
    assert cm.query(int(keys[0])) == 255                          # saturating
    for cls in (core.BloomFilter, core.BlockBloomFilter):
        bf = cls(1 << 16, 3)
        for k in keys[:1000].tolist():
            bf.insert(k)
        assert all(bf.query(k) for k in keys[:1000].tolist())
        assert sum(bf.query(k) for k in keys[1000:2000].tolist()) < 100
    bm = core.Bitmap(100, False)
    for i in (3, 17, 64, 99):
        bm.set(i)
    assert bm.nnz() == 4 and bm.test(64) and not bm.test(65)
    bm.clear(64); assert bm.nnz() == 3
    bm.fill(True); assert bm.nnz() == 100
    ff = core.FreqencyFilter(); ff.resize(1 << 14, 2)
    ff.insert_keys(keys[:100], np.full(100, 5, np.uint8)); ff.insert_keys(keys[:50], np.full(50, 5, np.uint8))
    kept = ff.query_keys(keys[:100], 7)
    assert set(keys[:50].tolist()) <= set(kept.tolist()) and len(kept) < 60


# ---------------------------------------------------------------- filters
def _msg(keys, vals, filters, channel=0, push=True):
    m = core.Message(core.request(channel, filters=filters))
    t = m.task; t.has_param = True; p = t.param; p.push = push; t.param = p; m.task = t
    m.set_key(np.asarray(keys, np.uint64))
    m.add_value(np.asarray(vals, np.float32))
    return m


def test_key_caching_filter_drops_repeated_keys():
    F = core.FilterConfig
    send, recv = core.FilterChain(), core.FilterChain()
    keys = np.arange(1, 1000, dtype=np.uint64) * 7
    sizes = []
    for it in range(3):
        m = _msg(keys, np.full(len(keys), float(it)), [F(F.Type.KEY_CACHING)])
        send.encode(m)
        sizes.append(m.key_bytes())
        recv.decode(m)
        assert np.array_equal(m.key(), keys) and m.value(0)[0] == it
    assert sizes == [len(keys) * 8, 0, 0]
    m = _msg(keys[:-1], np.zeros(len(keys) - 1), [F(F.Type.KEY_CACHING)])   # a different list: sent in full
    send.encode(m); assert m.key_bytes() == (len(keys) - 1) * 8
    recv.decode(m); assert np.array_equal(m.key(), keys[:-1])
    # a receiver that never saw the keys refuses a signature-only message
    m = _msg(keys[:-1], np.zeros(len(keys) - 1), [F(F.Type.KEY_CACHING)]); send.encode(m)
    with pytest.raises(core.CheckError):
        core.FilterChain().decode(m)


def test_compressing_and_fixing_float_filters():
    F = core.FilterConfig
    rng = np.random.default_rng(1)
    keys = np.sort(rng.integers(0, 1 << 30, 5000, dtype=np.uint64))
    vals = np.round(rng.normal(size=5000), 1).astype(np.float32)
    send, recv = core.FilterChain(), core.FilterChain()
    m = _msg(keys, vals, [F(F.Type.COMPRESSING)])
    raw = m.key_bytes() + m.value_bytes(0)
    send.encode(m)
    assert m.key_bytes() + m.value_bytes(0) < 0.7 * raw
    recv.decode(m)
    assert np.array_equal(m.key(), keys) and np.array_equal(m.value(0), vals)
    for nbytes in (1, 2, 3):
        send, recv = core.FilterChain(), core.FilterChain()
        send.set_fixing_float_seed(7)
        m = _msg(keys, vals, [F(F.Type.FIXING_FLOAT, num_bytes=nbytes), F(F.Type.COMPRESSING)])
        send.encode(m)
        recv.decode(m)
        step = (vals.max() + 1e-6 - vals.min()) / (2 ** (8 * nbytes) - 2)
        assert np.abs(m.value(0) - vals).max() <= step * 1.001 + 1e-6
    # an explicit range clamps
    f = F(F.Type.FIXING_FLOAT, num_bytes=2); f.set_range(-1.0, 1.0)
    m = _msg(keys[:4], [-5.0, -0.5, 0.5, 5.0], [f])
    c = core.FilterChain(); c.encode(m); c.decode(m)
    assert np.allclose(m.value(0), [-1, -0.5, 0.5, 1], atol=1e-3)
    m = _msg(keys[:1000], np.zeros(1000), [F(F.Type.NOISE, mean=2.0, std=0.5)])
    core.FilterChain().encode(m)
    assert abs(m.value(0).mean() - 2.0) < 0.1 and 0.4 < m.value(0).std() < 0.6
    v = core.sparse_filter_mark()
    assert v != v                                                       # the "inactive" mark is a NaN


# ---------------------------------------------------------------- parsers and readers
def test_text_parsers_all_formats():
    ex = core.parse_example("-1 2:0.5 9:1.5 100:2", "LIBSVM")
    assert ex[0]["val"].tolist() == [-1.0] and ex[1]["key"].tolist() == [2, 9, 100] and ex[1]["val"].tolist() == [0.5, 1.5, 2.0]
    assert core.parse_example("1 9:1 2:1", "LIBSVM") is None            # ids must ascend
    assert core.parse_example("x 1:1", "LIBSVM") is None
    ex = core.parse_example("1001 1 1 7:3 8:3 9:5", "ADFEA")
    assert ex[0]["val"].tolist() == [1.0] and ex[3]["key"].tolist() == [7, 8] and ex[5]["key"].tolist() == [9]
    ex = core.parse_example("1001 1 0 7:3 8:3 9:5", "ADFEA", True)
    assert ex[0]["val"].tolist() == [-1.0] and ex[1]["key"].tolist() == [7, 8, 9]
    g5, g9 = (5 << 54) | 123, (9 << 54) | 77
    ex = core.parse_example(f"1 88 | {g5} {g9} {g5 + 1}", "TERAFEA")
    assert ex[5]["key"].tolist() == [g5, g5 + 1] and ex[9]["key"].tolist() == [g9]
    ex = core.parse_example("1; 1 5 9; 3 7", "SPARSE_BINARY")
    assert ex[1]["key"].tolist() == [5, 9] and ex[3]["key"].tolist() == [7] and len(ex[1]["val"]) == 0
    ex = core.parse_example("0; 1 5:0.5 9:2", "SPARSE")
    assert ex[0]["val"].tolist() == [-1.0] and ex[1]["key"].tolist() == [5, 9] and ex[1]["val"].tolist() == [0.5, 2.0]
    ex = core.parse_example("1; 2 0.5 1.5 2.5", "DENSE")
    assert ex[2]["val"].tolist() == [0.5, 1.5, 2.5] and len(ex[2]["key"]) == 0
    cols = ["1"] + ["3", "", "7"] + [""] * 10 + ["68fd1e64", "abc", "a9d771cd", ""] + ["05db9164"] * 22
    ex = core.parse_example("\t".join(cols), "CRITEO")
    kmax = (1 << 64) - 1
    assert ex[1]["key"].tolist() == [3] and ex[3]["key"].tolist() == [kmax // 13 * 2 + 7]
    a, b = core.murmurhash3_x64_128(b"68fd1e64", 512927377)
    assert ex[14]["key"].tolist() == [a ^ b] and 15 not in ex                # short strings are skipped
    merged = core.parse_example("\t".join(cols), "CRITEO", True)
    assert sorted(merged) == [0, 1] and len(merged[1]["key"]) == 2 + 24


def test_stream_reader_slot_reader_and_recordio(tmp_path):
    rows = [f"{1 if i % 3 else -1}; 1 {i + 1} {i + 100}; 2 {i * 2 + 7};" for i in range(250)]
    f1, f2 = tmp_path / "part-0", tmp_path / "part-1.gz"
    f1.write_text("\n".join(rows[:100]) + "\n")
    with gzip.open(f2, "wt") as g:
        g.write("\n".join(rows[100:]) + "\n")
    files = core.search_files([str(tmp_path / "part-.*")])
    assert [os.path.basename(f) for f in files] == ["part-0", "part-1.gz"]
    r = core.StreamReader(files, "TEXT", "SPARSE_BINARY")
    y, mats = r.read_matrices(120)
    assert len(y) == 120 and y[0] == -1 and y[1] == 1
    assert [m["id"] for m in mats] == [1, 2] and mats[0]["offset"].tolist() == list(range(0, 241, 2))
    assert mats[0]["index"][:4].tolist() == [1, 100, 2, 101] and mats[0]["binary"]
    y2, _ = r.read_matrices(1000)
    assert len(y2) == 130 and r.read_matrices(10) is None
    r = core.StreamReader(files, "TEXT", "SPARSE_BINARY", True)        # feature groups merged
    _, mats = r.read_matrices(10)
    assert len(mats) == 1 and mats[0]["offset"].tolist() == list(range(0, 31, 3))
    r = core.StreamReader(files, "TEXT", "SPARSE_BINARY"); r.set_hash_kernel(16)
    _, mats = r.read_matrices(250)
    assert mats[0]["index"].max() < 16
    # record io: text -> records -> the same examples
    rec = str(tmp_path / "all.rec")
    assert core.text_to_records(files, "SPARSE_BINARY", rec) == 250
    y3, mats3 = core.StreamReader([rec], "PROTO", "SPARSE_BINARY").read_matrices(1000)
    assert len(y3) == 250 and mats3[1]["index"][-1] == 249 * 2 + 7
    # slot reader: column arrays per slot, cached on disk
    cache = str(tmp_path / "cache")
    sr = core.SlotReader(files, "SPARSE_BINARY", cache)
    info = sr.read(2)
    assert info["num_ex"] == 250 and {s["id"]: s["nnz_ele"] for s in info["slot"]} == {0: 250, 1: 500, 2: 250}
    assert not sr.hit_cache() and sr.offset(1).tolist() == list(range(0, 501, 2)) and len(sr.index(2)) == 250
    assert sr.value(0)[:3].tolist() == [-1.0, 1.0, 1.0]
    sr2 = core.SlotReader(files, "SPARSE_BINARY", cache)
    sr2.read(2)
    assert sr2.hit_cache() and np.array_equal(sr2.index(1), sr.index(1))


def test_localizer_spmv_transpose_evaluation():
    rng = np.random.default_rng(2)
    rows, z = 50, 6
    idx = rng.integers(0, 1 << 60, 40, dtype=np.uint64)[rng.integers(0, 40, rows * z)]
    off = np.arange(rows + 1, dtype=np.uint64) * z
    uniq, cnt, col = core.localize(off, idx)
    u, inv, c = np.unique(idx, return_inverse=True, return_counts=True)
    assert np.array_equal(uniq, u) and np.array_equal(cnt, c) and np.array_equal(col, inv)
    x = rng.normal(size=len(u)).astype(np.float32)
    val = rng.random(rows * z, dtype=np.float32)
    dense = np.zeros((rows, len(u)), np.float32)
    np.add.at(dense, (np.repeat(np.arange(rows), z), inv), val)
    assert np.allclose(core.spmv(off, col, val, x, len(u)), dense @ x, atol=1e-4)
    g = rng.normal(size=rows).astype(np.float32)
    assert np.allclose(core.spmv(off, col, val, g, len(u), True, 3), dense.T @ g, atol=1e-4)
    binary = (dense != 0)
    t_off, t_idx = core.transpose_csr(off, col, len(u))
    assert np.array_equal(np.diff(t_off.astype(np.int64)), np.bincount(inv, minlength=len(u)))
    assert all(binary[t_idx[t_off[j]:t_off[j + 1]], j].all() for j in range(len(u)))
    y = np.where(rng.random(500) < 0.4, 1, -1).astype(np.float32)
    s = (y * 0.7 + rng.normal(size=500)).astype(np.float32)
    ev = core.evaluate(y, s)
    from parameter_server_b200.utils.oracle import auc
    assert abs(ev["auc"] - auc(y, s)) < 1e-6 and abs(ev["auc_histogram"] - ev["auc"]) < 5e-3
    assert abs(ev["logloss"] - np.mean(np.log1p(np.exp(-y * s)))) < 1e-5
    assert abs(ev["accuracy"] - np.mean((s > 0) == (y > 0))) < 1e-6
    n, out = core.ordered_match(np.array([1, 5, 9], np.uint64), np.array([1, 2, 3], np.float32),
                                np.array([0, 5, 9, 11], np.uint64), np.zeros(4, np.float32), 1, 1, 2)
    assert n == 2 and out.tolist() == [0, 2, 3, 0]
    assert core.parallel_sort_u64(np.array([5, 1, 9, 3], np.uint64), 2).tolist() == [1, 3, 5, 9]


# ---------------------------------------------------------------- control-plane helpers
def test_options_env_workload_pool_dashboard(tmp_path, monkeypatch):
    o = core.Options.parse(["-num_servers", "2", "--num_workers=3", "-my_node", "role:WORKER,hostname:'h',port:9,id:'W7'",
                            "-local", "-app_file", "x.conf", "-key_end", "1000", "positional"])
    assert (o.num_servers, o.num_workers, o.local, o.app_file, o.key_end, o.rest) == (2, 3, True, "x.conf", 1000, ["positional"])
    n = core.parse_node(o.my_node)
    assert (n.role, n.hostname, n.port, n.id) == (core.Node.Role.WORKER, "h", 9, "W7")
    assert core.parse_node("role:SERVER,hostname:'10.0.0.1',port:80").id == "S_10.0.0.1_80"
    for k, v in dict(DMLC_PS_ROOT_URI="10.1.1.1", DMLC_PS_ROOT_PORT="8000", DMLC_NUM_WORKER="4", DMLC_NUM_SERVER="2",
                     DMLC_ROLE="server").items():
        monkeypatch.setenv(k, v)
    o = core.Options(); o.init_from_env()
    assert o.num_workers == 4 and "10.1.1.1" in o.scheduler and core.parse_node(o.my_node).role == core.Node.Role.SERVER
    monkeypatch.delenv("DMLC_ROLE"); monkeypatch.setenv("OMPI_COMM_WORLD_RANK", "3")
    o = core.Options(); o.init_from_env()
    assert core.parse_node(o.my_node).role == core.Node.Role.WORKER       # ranks 1..2 are servers, 3.. workers
    files = []
    for i in range(3):
        p = tmp_path / f"d{i}"; p.write_text("x"); files.append(str(p))
    pool = core.WorkloadPool(files, replica=2)
    assert pool.size() == 6
    a = [pool.assign("W0") for _ in range(2)]; b = pool.assign("W1")
    pool.finish(a[0][0]); pool.restore("W0")                              # W0 dies with one workload unfinished
    assert pool.assign("W1")[0] == a[1][0] and pool.num_finished() == 1
    hb = core.HeartbeatInfo(); hb.init("", "host-a"); hb.increase_in_bytes(5 << 20)
    d = core.Dashboard(); d.add_task("W1", 7); d.add_report("W1", hb.get()); d.add_report("H", hb.get()); d.add_report("S0", hb.get())
    rep = d.report().splitlines()
    assert "busy(ms)" in rep[0] and [l.split()[0] for l in rep[1:]] == ["H", "S0", "W1"] and " 7 " in rep[3]
    tt = core.TaskTracker(); tt.start(1); assert tt.was_started(1) and not tt.has_finished(1)
    tt.finish(1); tt.wait(1); assert tt.has_finished(1)


def test_checkpoint_file_roundtrip(tmp_path):
    """Binary shard checkpoint: what is written is read back bit for bit; bad files are refused."""
    import numpy as np
    import pytest
    from parameter_server_b200.utils import checkpoint as ck
    rng = np.random.default_rng(0)
    n = 1000
    keys = np.sort(rng.integers(0, 1 << 63, n, dtype=np.uint64))
    w, s0, s1 = (rng.standard_normal(n).astype(np.float32) for _ in range(3))
    p = ck.shard_path(str(tmp_path / "m"), 3)
    ck.write_shard(p, keys, w, s0, s1, {"rank": 3, "world": 4, "key_begin": 0, "key_end": 1 << 63, "meta": {"step": 17}})
    hdr, k2, w2, a2, b2 = ck.read_shard(p)
    assert hdr["n"] == n and hdr["meta"]["step"] == 17 and hdr["rank"] == 3
    assert np.array_equal(k2, keys) and np.array_equal(w2, w) and np.array_equal(a2, s0) and np.array_equal(b2, s1)
    bad = tmp_path / "bad.psbckpt"
    bad.write_bytes(b"not a checkpoint")
    with pytest.raises(ValueError):
        ck.read_shard(str(bad))
    blob = open(p, "rb").read()
    trunc = tmp_path / "trunc.psbckpt"
    trunc.write_bytes(blob[:len(blob) - 100])
    with pytest.raises(ValueError):
        ck.read_shard(str(trunc))


def test_s3_files_are_read_through_curl(tmp_path, monkeypatch):
    """s3://bucket/object is read from a `curl` pipe (a stand-in curl here: no network), bucket
    listings expand a file-name pattern, and nothing but plain characters reaches the shell."""
    import os
    import stat
    from parameter_server_b200.system import core
    store = tmp_path / "bucket"
    (store / "data").mkdir(parents=True)
    (store / "data" / "part-0").write_text("1 3:1 7:1\n")
    (store / "data" / "part-1").write_text("-1 2:1\n")
    fake = tmp_path / "bin" / "curl"
    fake.parent.mkdir()
    fake.write_text(f"""#!/bin/sh
url="$5"
case "$url" in
  *'?prefix='*) echo '<ListBucketResult><Contents><Key>data/part-0</Key></Contents><Contents><Key>data/part-1</Key></Contents><Contents><Key>data/other</Key></Contents></ListBucketResult>' ;;
  *) path="${{url#http://mybucket.s3.amazonaws.com/}}"; [ -f "{store}/$path" ] || exit 22; cat "{store}/$path" ;;
esac
""")
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{fake.parent}:{os.environ['PATH']}")
    assert core.s3_file_url("s3://mybucket/data/part-0") == "http://mybucket.s3.amazonaws.com/data/part-0"
    assert core.read_file("s3://mybucket/data/part-0") == b"1 3:1 7:1\n"
    assert core.search_files(["s3://mybucket/data/part-.*"]) == ["s3://mybucket/data/part-0", "s3://mybucket/data/part-1"]
    r = core.StreamReader(["s3://mybucket/data/part-1"], "TEXT", "LIBSVM", True)
    y, mats = r.read_matrices(10)
    assert list(y) == [-1.0] and list(mats[0]["index"]) == [2]
    assert core.read_file("s3://mybucket/data/x;rm -rf y") is None      # refused before any shell sees it


def _fake_hadoop(home, log):
    """<home>/bin/hadoop: `fs [-D k=v]... -cat URI` prints the local file behind hdfs://<path>, `-ls URI`
    prints a listing in the 8 columns of `hadoop fs -ls` (with a directory and a header line)."""
    import stat
    exe = home / "bin" / "hadoop"
    exe.parent.mkdir(parents=True)
    exe.write_text(f"""#!/bin/sh
echo "$@" >> {log}
[ "$1" = fs ] || exit 2
shift
while [ "$1" = -D ]; do shift; shift; done
op="$1"; path="${{2#hdfs://}}"
case "$op" in
  -cat) [ -f "$path" ] || exit 1; cat "$path" ;;
  -ls) echo "Found some items"
       echo "drwxr-xr-x   - u g          0 2015-03-18 16:34 $path/sub"
       for f in "$path"/*; do [ -f "$f" ] && echo "-rw-r--r--   3 u g       1234 2015-03-18 16:34 $f"; done ;;
  *) exit 2 ;;
esac
""")
    exe.chmod(exe.stat().st_mode | stat.S_IEXEC)


def test_hdfs_files_are_read_through_hadoop_fs(tmp_path):
    """A data block with `hdfs {{ home ugi namenode }}` names HDFS files: directories are listed with
    `hadoop fs -ls`, files are read from a `hadoop fs -cat` pipe (gunzip behind it for .gz), the -D options
    carry the name node and the user (a stand-in hadoop command here)."""
    import gzip
    from parameter_server_b200.system import core
    store = tmp_path / "store" / "train"
    (store / "sub").mkdir(parents=True)
    (store / "part-0").write_text("1 3:1 7:1\n")
    (store / "part-1").write_text("-1 2:1\n")
    with gzip.open(store / "zipped-0.gz", "wt") as f:
        f.write("1 5:1\n-1 6:1\n")
    (store / "other").write_text("x\n")
    log = tmp_path / "hadoop.log"
    _fake_hadoop(tmp_path / "hadoop", log)
    hdfs = {"home": str(tmp_path / "hadoop"), "ugi": "me,secret", "namenode": "nn:9000"}
    files = core.search_files([f"{store}/part-.*"], hdfs)
    assert files == [f"hdfs://{store}/part-0", f"hdfs://{store}/part-1"]
    assert core.hadoop_fs() == f"{tmp_path}/hadoop/bin/hadoop fs -D fs.default.name=nn:9000 -D hadoop.job.ugi=me,secret"
    assert core.read_file(files[0]) == b"1 3:1 7:1\n"
    y, mats = core.StreamReader([files[1]], "TEXT", "LIBSVM", True).read_matrices(10)
    assert list(y) == [-1.0] and list(mats[0]["index"]) == [2]
    y, mats = core.StreamReader([f"hdfs://{store}/zipped-0.gz"], "TEXT", "LIBSVM", True).read_matrices(10)
    assert list(y) == [1.0, -1.0] and list(mats[0]["index"]) == [5, 6]
    calls = log.read_text().splitlines()
    assert calls[0] == f"fs -D fs.default.name=nn:9000 -D hadoop.job.ugi=me,secret -ls hdfs://{store}"
    assert f"fs -D fs.default.name=nn:9000 -D hadoop.job.ugi=me,secret -cat hdfs://{store}/part-0" in calls
    assert core.read_file(f"hdfs://{store}/x;rm -rf y") is None      # refused before any shell sees it
    # the GPU application resolves a configuration's data block the same way
    from parameter_server_b200.app.linear import _files
    conf = core.parse_text_proto(f'training_data {{ hdfs {{ home: "{tmp_path}/hadoop" }} file: "{store}/part-.*" }}')
    assert _files(conf["training_data"]) == files


def test_data_tool_show_and_convert(tmp_path, capsys):
    """utils/datatool: `show` prints parsed examples, `convert` writes a record file that the stream reader
    reads back with format PROTO, and the per-slot statistics beside it."""
    import json
    from parameter_server_b200.system import core
    from parameter_server_b200.utils import datatool
    (tmp_path / "part-0").write_text("1 3:1 7:0.5\n-1 2:1\n")
    (tmp_path / "part-1").write_text("1 9:2\n")
    assert datatool.main(["show", "-input", str(tmp_path / "part-0"), "-format", "libsvm", "-n", "1"]) == 0
    first = json.loads(capsys.readouterr().out.strip())
    assert first["0"]["val"] == [1.0] and first["1"]["key"] == [3, 7] and first["1"]["val"] == [1.0, 0.5]
    assert datatool.main(["convert", "-input", str(tmp_path / "part-.*"), "-output", str(tmp_path / "all")]) == 0
    assert "3 examples from 2 file(s)" in capsys.readouterr().out
    info = json.load(open(tmp_path / "all.info"))
    assert info["num_ex"] == 3 and info["slot"][1]["nnz_ele"] == 4
    y, mats = core.StreamReader([str(tmp_path / "all.recordio")], "PROTO", "LIBSVM").read_matrices(10)
    assert list(y) == [1.0, -1.0, 1.0] and list(mats[0]["index"]) == [3, 7, 2, 9]


def test_resource_usage_and_matrix_debug_string():
    from parameter_server_b200.system import core
    r = core.res_usage()
    assert 1 < r["my_phy_mem_mb"] <= r["my_vir_mem_mb"]
    assert 0 < r["host_in_use_mem_mb"] < r["host_total_mem_mb"] and r["my_phy_mem_mb"] < r["host_total_mem_mb"]
    s = core.sparse_debug_string(np.array([0, 2, 3], np.uint64), np.array([1, 4, 2], np.uint32), None, 5)
    assert "SPARSE_BINARY row-major" in s and "nnz 3" in s and "index: [3]{1,4,2}" in s and "value" not in s
    s = core.sparse_debug_string(np.array([0, 2, 3], np.uint64), np.array([1, 4, 2], np.uint32),
                                 np.array([.5, 1, 2], np.float32), 5)
    assert "value: [3]{0.5,1,2}" in s


def test_reader_flags_in_process(tmp_path):
    """set_reader_flags: what -hash_kernel and -line_limit do to a stream reader made afterwards."""
    from parameter_server_b200.system import core
    f = tmp_path / "part-0"
    f.write_text("".join(f"1 {100 + i}:1 {200 + i}:1\n" for i in range(20)))
    try:
        core.set_reader_flags(hash_kernel=7, line_limit=5)
        y, mats = core.StreamReader([str(f)], "TEXT", "LIBSVM", True).read_matrices(100)
        assert len(y) == 5 and max(mats[0]["index"]) < 7
    finally:
        core.set_reader_flags()
    y, mats = core.StreamReader([str(f)], "TEXT", "LIBSVM", True).read_matrices(100)
    assert len(y) == 20 and max(mats[0]["index"]) == 219


def test_cycle_counter_timer_pair_moves_forward():
    """hwtic / hwtoc (the reference's cycle-counter timers, util/resource_usage.h): monotone and non-zero."""
    from parameter_server_b200.system import core
    t0 = core.hwtic()
    x = sum(range(20000))
    assert x > 0 and core.hwtoc(t0) > 0 and core.hwtic() >= t0
