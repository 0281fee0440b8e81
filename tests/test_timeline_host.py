"""The table that ``qwen_engine_b200.engine.timeline`` makes of a step's events, on made-up events (CPU)."""
from qwen_engine_b200.engine.timeline import layer_table


def _launch(file, line_start, line_wait, grid, t_start, t_wait):
    ev = []
    for cta in range(grid):
        ev.append((file, line_start, 0, cta, grid, t_start + 10 * cta, cta % 4))
        ev.append((file, line_wait, 1, cta, grid, t_wait + 10 * cta, cta % 4))
    return ev


def test_layer_table_groups_the_events_between_two_attention_launches():
    ev = []
    for layer in range(3):
        base = 100_000 * layer
        ev += _launch("attention_decode_mma.cu", 63, 142, 4, base, base + 5_000)
        ev += _launch("gemm_small_m.cu", 49, 50, 2, base + 6_000, base + 16_000)
        ev += _launch("elementwise.cu", 151, 164, 1, base + 17_000, base + 20_000)
    ev.sort(key=lambda e: e[5])
    text = layer_table(ev, 1)
    lines = text.splitlines()
    assert "100.00 us from attention launch 1 to the next" in lines[0] and "3 launches of 4 CTAs" in lines[0]
    rows = {(l.split()[0], " ".join(l.split()[1:3])): l.split() for l in lines[2:]}
    att = rows[("attention_decode_mma.cu:63", "CTA started")]
    assert att[3:5] == ["4", "4"] and float(att[5]) == 0.0 and float(att[7]) == 0.03
    wait = rows[("gemm_small_m.cu:50", "wait returned")]
    assert wait[3:5] == ["2", "2"] and float(wait[5]) == 16.0
    assert ("elementwise.cu:164", "wait returned") in rows
    # nothing of the other layers: every probe has as many events as its grid
    assert all(int(r[4]) == int(r[3]) for r in rows.values())


def test_layer_table_without_attention_launches():
    assert "no attention launches" in layer_table([("gemm_small_m.cu", 49, 0, 0, 1, 5, 0)], 0)
