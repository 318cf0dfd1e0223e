"""alpha-beta fit and bucket arithmetic (FINAL_CLEAN_CODE_/scripts/predict_comm_model.py:14-18,109-139)."""
from cme213_final_project_b200.parallel import comm_model as cm


def test_fit_recovers_line():
    pts = [(b, 0.02 + 3e-9 * b) for b in (4096, 65536, 1 << 20, 1 << 25)]
    a, b = cm.fit_alpha_beta(pts)
    assert abs(a - 0.02) < 1e-9 and abs(b - 3e-9) < 1e-15
    assert abs(cm.predict_bucketed(a, b, [1 << 20] * 8) - (8 * 0.02 + 3e-9 * (8 << 20))) < 1e-9


def test_reference_gradient_sizes():
    assert cm.gradient_floats(128, 512, 65, 64) == 222592
    assert cm.gradient_floats(256, 1024, 65, 64) == 838400
    assert cm.gradient_floats(512, 2048, 65, 64) == 3249664


def test_shard_alignment_makes_every_bucket_split_for_any_world():
    """Arena alignment lcm(64, 8 * world): every natural and coalesced bucket divides into `world` slices of whole
    16-byte bf16 vectors, also for worlds of 3, 5, 6, 7 (the reference validates 3 ranks,
    FINAL_CLEAN_CODE_/scripts/run_edge_case_validation.sh:90-97) and for shapes with odd extents (vocabulary 65)."""
    from cme213_final_project_b200.arena import ArenaLayout
    from cme213_final_project_b200.config import min_bucket_elems, preset
    from cme213_final_project_b200.parallel.fused_sync import shard_align
    assert [shard_align(w) for w in (1, 2, 3, 4, 5, 6, 7, 8, 16)] == [64, 64, 192, 64, 320, 192, 448, 64, 128]
    for name in ("tiny-gpt", "parity-h128", "char-gpt"):
        cfg, _ = preset(name)
        for world in range(1, 9):
            lay = ArenaLayout(cfg, align=shard_align(world))
            for kb in (0, 64, 1024):
                for b in lay.coalesced_buckets(min_bucket_elems(kb, 2)):
                    assert b.numel % (8 * world) == 0 and b.start % 8 == 0, (name, world, kb, b)
            assert lay.num_params() == ArenaLayout(cfg, align=64).num_params()


def test_algorithm_choice_follows_the_measured_table():
    from cme213_final_project_b200.parallel.fused_sync import choose_algo, load_table, table_for_world
    table = load_table()
    assert {"2", "8"} <= set(table)
    t8, t2 = table_for_world(table, 8), table_for_world(table, 2)
    assert choose_algo(64 << 20, 8, True, t8) == "nvls"
    assert choose_algo(64 << 10, 8, True, t8) == "two_shot"          # below the measured NVLS crossover
    assert choose_algo(64 << 20, 8, False, t8) == "two_shot"         # no multicast mapping
    assert choose_algo(64 << 20, 2, True, t2) == "two_shot"          # in-switch reduction never won at 2 ranks
    assert choose_algo(1024, 8, True, {"one_shot_max_bytes": 4096}) == "one_shot"
    assert table_for_world(table, 7) is t8 and table_for_world(table, 3) in (t2, table_for_world(table, 4))
    assert table_for_world({}, 4) == {}
