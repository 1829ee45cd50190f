"""The ncu report reducer on a synthetic raw-page CSV."""
from tileccl_b200.bench import ncu_summary


def test_summary_picks_metrics_and_top_stalls():
    rows = [
        ["ID", "Kernel Name", "gpu__time_duration.sum", "dram__bytes_read.sum", "launch__registers_per_thread",
         "smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio", "smsp__average_warps_issue_stalled_wait_per_issue_active.ratio", "other"],
        ["", "", "us", "Mbyte", "register/thread", "inst", "inst", ""],
        ["0", "k<1>", "10.0", "5", "32", "1.5", "0.2", "x"],
        ["1", "k<2>", "692.5", "1039", "168", "11.46", "2.39", "y"],
    ]
    txt = ncu_summary.summarize(rows)
    assert "k<2>" in txt and "k<1>" not in txt
    assert "| gpu__time_duration.sum | 692.5 us |" in txt and "| launch__registers_per_thread | 168 register/thread |" in txt
    assert "barrier 11.46, wait 2.39" in txt
    assert "k<1>" in ncu_summary.summarize(rows, all_launches=True)
    assert "no launches" in ncu_summary.summarize(rows[:2])
