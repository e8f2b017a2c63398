

def test_stream_stages_split_limit_and_read_files(tmp_path):
    from torchrec_b200.datasets.utils import Limit, LoadFiles, ParallelReadConcat, ReadLinesFromCSV, idx_split_train_val, rand_split_train_val, safe_cast

    assert safe_cast("7", int, 0) == 7 and safe_cast("", int, -1) == -1
    data = list(range(1000))
    train, val = idx_split_train_val(data, 0.75)
    t, v = list(train), list(val)
    assert len(t) == 750 and sorted(t + v) == data and list(train) == t  # exact proportion, disjoint, re-iterable
    rt, rv = rand_split_train_val(data, 0.7, random_seed=3)
    a, b = list(rt), list(rv)
    assert sorted(a + b) == data and 620 < len(a) < 780 and list(rt) == a
    assert list(Limit(data, 5)) == [0, 1, 2, 3, 4]
    files = []
    for i in range(3):
        p = tmp_path / f"part{i}.tsv"
        p.write_text("h1\th2\n" + "".join(f"{i}\t{j}\n" for j in range(4)))
        files.append(str(p))
    rows = list(ReadLinesFromCSV(LoadFiles(files, mode="t"), skip_first_line=True, delimiter="\t"))
    assert len(rows) == 12 and rows[0] == ["0", "0"] and rows[-1] == ["2", "3"]
    pipes = [ReadLinesFromCSV(LoadFiles([f], mode="t"), skip_first_line=True, delimiter="\t") for f in files]
    assert list(ParallelReadConcat(*pipes)) == rows
