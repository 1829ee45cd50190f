"""Parsers of the reference movers' stdout tables (formats: tests/pk_bw_sweep.cu:739-826,
tests/p2p_ce_vs_tma.cu:774-789 of the reference), on text made with the same printf formats."""
from tileccl_b200.bench import ref_movers as R


def _cell(g, flag=" "):
    return " %11.2f%c" % (g, flag)


def test_parse_fig2_and_fig3():
    text = "=== PK transfer-mechanism sweep (paper Fig.2 / Fig.3) ===\nmax opt-in shared memory / CTA: 232448 B\n\n"
    text += "--- Fig.2: bandwidth (GB/s) vs message size   [blocks=148, stages<=4] ---\n"
    text += "%-10s %12s %12s %12s\n" % ("msg_size", "ce", "tma", "reg")
    text += "%-10s" % "128 B" + _cell(0.04, "*") + _cell(77.97) + _cell(625.81) + "\n"
    text += "%-10s" % "8 KiB" + _cell(2.5, "*") + _cell(690.1) + _cell(697.0) + "\n"
    text += "%-10s" % "128 MiB" + _cell(748.0) + " %11s " % "-" + _cell(696.5, "!") + "\n"
    text += "flags: * ce payload capped\n\n"
    text += "--- Fig.3: bandwidth (GB/s) vs SM count   [msg: tma=56 KiB, reg=16 KiB, reg_threads=1024] ---\n"
    text += "copy-engine reference (1 call, 256 MiB, 0 SMs): 750.12 GB/s\n"
    text += "%-6s %12s %12s\n" % ("sms", "tma", "reg")
    text += "%-6d" % 1 + _cell(55.5) + _cell(48.25) + "\n"
    text += "%-6d" % 16 + _cell(690.0, "^") + _cell(688.0) + "\n"
    text += "flags: ^ tma single-buffer\n"
    f2 = R.parse_pk_fig2(text)
    assert f2[("ce", 128)] == 0.04 and f2[("tma", 128)] == 77.97 and f2[("reg", 8192)] == 697.0
    assert f2[("ce", 128 << 20)] == 748.0 and ("tma", 128 << 20) not in f2 and f2[("reg", 128 << 20)] == 696.5
    f3 = R.parse_pk_fig3(text)
    assert f3 == {("tma", 1): 55.5, ("reg", 1): 48.25, ("tma", 16): 690.0, ("reg", 16): 688.0}


def test_parse_token_blocks():
    text = "--- tokens=64   payload=0.875 MiB   tile=14336 B (1 tok)   tiles=64   stages=4   blocks=64   smem=57376 B ---\n"
    text += "%-11s %12s %12s %12s %12s %8s\n" % ("method", "avg(us)", "p50(us)", "p99(us)", "BW(GB/s)", "verify")
    text += "%-11s %12.2f %12.2f %12.2f %12.2f %8s\n" % ("ce", 4.5, 7.0, 7.5, 203.9, "ok")
    text += "%-11s %12s %12s %12s %12s %8s  %s\n" % ("tma_pull", "-", "-", "-", "-", "-", "failed")
    text += "%-11s %12.2f %12.2f %12.2f %12.2f %8s\n" % ("sm_pull", 6.25, 11.0, 14.0, 146.8, "ok")
    text += "\n--- tokens=4096   payload=56.000 MiB   tile=57344 B (4 tok)   tiles=1024   stages=4   blocks=148   smem=229408 B ---\n"
    text += "%-11s %12s %12s %12s %12s %8s\n" % ("method", "avg(us)", "p50(us)", "p99(us)", "BW(GB/s)", "verify")
    text += "%-11s %12.2f %12.2f %12.2f %12.2f %8s\n" % ("tma", 84.1, 90.0, 95.5, 698.2, "ok")
    p = R.parse_p2p(text)
    assert p[("ce", 64)] == (4.5, 203.9) and p[("sm_pull", 64)] == (6.25, 146.8) and ("tma_pull", 64) not in p
    assert p[("tma", 4096)] == (84.1, 698.2)


def test_sizes():
    assert R.parse_size("128 B") == 128 and R.parse_size("8 KiB") == 8192 and R.parse_size("1 GiB") == 1 << 30
