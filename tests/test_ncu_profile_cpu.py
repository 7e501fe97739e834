"""The Nsight Compute summary reader on a synthetic `--page raw --csv` table (no GPU, no ncu needed)."""
from gpu_kernels_b200 import ncu_profile as P

RAW = '''"ID","Process ID","Kernel Name","gpu__time_duration.sum","dram__bytes_read.sum","launch__grid_size","smsp__average_warps_issue_stalled_barrier_per_issue_active.ratio","smsp__average_warps_issue_stalled_long_scoreboard_per_issue_active.ratio","smsp__average_warps_issue_stalled_selected_per_issue_active.ratio"
"","","","us","Mbyte","","inst","inst","inst"
"0","77","quantise_kernel<__nv_bfloat16, 256>(const T1 *)","34.5","134.2","2048","0.4","6.2","1.0"
"1","77","quantise_kernel<__nv_bfloat16, 256>(const T1 *)","34.9","134.2","2048","0.5","6.0","1.0"
'''


def test_reads_every_launch_and_ranks_the_stalls():
    launches = P.read_raw_csv(RAW)
    assert len(launches) == 2
    assert launches[1]["gpu__time_duration.sum"] == ("34.9", "us")
    summary = dict(P.summarise(launches[0]))
    assert summary["duration"] == "34.5 us" and summary["DRAM read"] == "134.2 Mbyte" and summary["grid"] == "2048"
    assert summary["top warp stalls per issue"] == "long_scoreboard 6.2, barrier 0.4"      # 'selected' is not a stall
    assert summary["kernel"].startswith("quantise_kernel")


def test_an_empty_or_foreign_table_gives_nothing():
    assert P.read_raw_csv("") == [] and P.read_raw_csv("==PROF== no kernels\n") == []
