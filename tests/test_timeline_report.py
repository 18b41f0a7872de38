"""The step timeline's grouping of marks into launches (`csrc/timeline.py`), on made-up marks."""
from ember_cpp_b200.csrc.timeline import launches_of, report


def marks_of(kernel, grid, start, blocks=None, dep=None, end=None, sms=148):
    """Block b runs on SM b % sms."""
    out = []
    for b in (range(grid) if blocks is None else blocks):
        out.append((start + b, kernel, 0, b, grid, b % sms))
        if dep is not None:
            out.append((dep + b, kernel, 1, b, grid, b % sms))
        if end is not None:
            out.append((end + 2 * b, kernel, 2, b, grid, b % sms))
    return out


def test_marks_are_grouped_into_launches():
    marks = (marks_of("layernorm", 8, 1000, dep=3000, end=5000, sms=3)
             + marks_of("linear_decode", 4, 2000, dep=6000, end=8000)
             # a kernel whose idle blocks leave no mark: two launches of the same grid, told apart by a block that repeats
             + marks_of("attention_decode", 16, 9000, blocks=(0, 1, 5), dep=9500, end=11000)
             + marks_of("attention_decode", 16, 20000, blocks=(0, 1, 2, 5), dep=20500, end=22000)
             + marks_of("linear_decode", 4, 30000, dep=31000, end=32000))
    marks.sort()
    launches = launches_of(marks)
    assert [(x["kernel"], x["grid"], x["n"]) for x in launches] == [
        ("layernorm", 8, 8), ("linear_decode", 4, 4), ("attention_decode", 16, 3), ("attention_decode", 16, 4),
        ("linear_decode", 4, 4)]
    assert launches[0]["t"][0] == (1000, 1007) and launches[0]["t"][1] == (3000, 3007) and launches[0]["t"][2] == (5000, 5014)
    assert launches[3]["blocks"][5] == {0: 20005, 1: 20505, 2: 22010}
    text = report(launches, "attention_decode")
    lines = text.split("\n")
    assert lines[0].startswith("layernorm") and "dep    2.00..   2.01" in lines[0]
    assert "on   3 SMs (<=  3)" in lines[0] and "on   4 SMs (<=  1)" in lines[1]   # 8 blocks on 3 SMs: 3, 3 and 2
    assert sum(1 for line in lines if line.startswith("block")) == 4      # every block of the kernel's last launch here
