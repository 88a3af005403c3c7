"""Puzzle definitions from files (mgt_load_puzzle_definition) against the reference's LoadPuzzleDefinition
(native/src/puzzle_io.cpp:48-97) and the reference's own test (native/tests/test_puzzle_io.cpp): host code only."""
import json

import numpy as np
import pytest

import multigputrainmlp_b200 as mgt

OK, INVALID_PUZZLE, IO_FAILURE = 0, 2, 6


def write_puzzle(tmp_path, moves, target, name="p", group_id=888, state_len=72, move_count=18):
    path = tmp_path / f"{name}.json"
    path.write_text(json.dumps({"group_id": group_id, "state_len": state_len, "move_count": move_count,
                                "moves": [[int(v) for v in m] for m in moves]}, indent=1))
    tpath = tmp_path / f"{name}-target.bin"
    tpath.write_bytes(bytes(int(v) for v in target))
    return path, tpath


def random_puzzle(seed, state_len=72, move_count=18):
    rng = np.random.default_rng(seed)
    return [rng.permutation(state_len) for _ in range(move_count)], rng.integers(0, 72, state_len)


def test_identity_fixture_as_in_the_reference_test(tmp_path, reference):
    # the reference's fixture holds 18 identity permutations and the identity target (native/tests/fixtures)
    jp, tp = write_puzzle(tmp_path, [np.arange(72)] * 18, np.arange(72))
    st, moves, target = mgt.load_puzzle_definition(jp, tp)
    assert st == OK
    assert np.array_equal(target[:72], np.arange(72)) and not target[72:].any()        # test_puzzle_io.cpp:14-17
    assert np.array_equal(moves[0], np.arange(80))                                    # pad positions map to themselves (:18)
    if reference is not None:
        rst, rmoves, rtarget = reference.load_puzzle(jp, tp)
        assert rst == OK and np.array_equal(rmoves, moves) and np.array_equal(rtarget, target)


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_random_permutations_match_the_reference_loader(tmp_path, reference, seed):
    perms, tgt = random_puzzle(seed)
    jp, tp = write_puzzle(tmp_path, perms, tgt)
    st, moves, target = mgt.load_puzzle_definition(jp, tp)
    assert st == OK
    for k in range(18):
        assert np.array_equal(moves[k, :72], perms[k]) and np.array_equal(moves[k, 72:], np.arange(72, 80))
    assert np.array_equal(target[:72], tgt) and not target[72:].any()
    if reference is not None:
        rst, rmoves, rtarget = reference.load_puzzle(jp, tp)
        assert rst == OK and np.array_equal(rmoves, moves) and np.array_equal(rtarget, target)


def test_rejections_carry_the_reference_status(tmp_path, reference):
    perms, tgt = random_puzzle(9)
    good_json, good_target = write_puzzle(tmp_path, perms, tgt, "good")
    cases = {}
    bad = [p.copy() for p in perms]
    bad[0][1] = bad[0][0]                                   # test_puzzle_io.cpp:21-41: a repeated value is not a permutation
    cases["repeat"] = (write_puzzle(tmp_path, bad, tgt, "repeat")[0], good_target, INVALID_PUZZLE)
    big = [p.copy() for p in perms]
    big[3][5] = 72
    cases["range"] = (write_puzzle(tmp_path, big, tgt, "range")[0], good_target, INVALID_PUZZLE)
    cases["group"] = (write_puzzle(tmp_path, perms, tgt, "group", group_id=887)[0], good_target, INVALID_PUZZLE)
    cases["short"] = (write_puzzle(tmp_path, perms[:17], tgt, "short")[0], good_target, INVALID_PUZZLE)
    short_t = tmp_path / "short-target.bin"
    short_t.write_bytes(bytes(71))
    cases["target71"] = (good_json, short_t, INVALID_PUZZLE)
    long_t = tmp_path / "long-target.bin"
    long_t.write_bytes(bytes(73))
    cases["target73"] = (good_json, long_t, INVALID_PUZZLE)
    cases["nojson"] = (tmp_path / "missing.json", good_target, IO_FAILURE)
    cases["notarget"] = (good_json, tmp_path / "missing.bin", IO_FAILURE)
    for name, (jp, tp, want) in cases.items():
        st, _, _ = mgt.load_puzzle_definition(jp, tp)
        assert st == want, name
        if reference is not None:
            assert reference.load_puzzle(jp, tp)[0] == want, name


def test_smaller_puzzles_are_arguments_here(tmp_path):
    # the reference fixes 888 / 72 / 18; the library takes them as arguments (unused move records are identities)
    perms, tgt = random_puzzle(4, state_len=24, move_count=6)
    jp, tp = write_puzzle(tmp_path, perms, tgt % 24, "small", group_id=7, state_len=24, move_count=6)
    st, moves, target = mgt.load_puzzle_definition(jp, tp, group_id=7, state_len=24, move_count=6)
    assert st == OK
    assert np.array_equal(moves[5, :24], perms[5]) and np.array_equal(moves[5, 24:], np.arange(24, 80))
    assert np.array_equal(moves[6], np.arange(80)) and not target[24:].any()
    assert mgt.load_puzzle_definition(jp, tp)[0] == INVALID_PUZZLE  # defaults expect 888 / 72 / 18
