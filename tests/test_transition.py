"""Transition detector against a line-by-line replay of the reference driver's state machine
(main_conv_ff.py:211-242)."""
import torch

from spion_b200.transition import TransitionDetector


def reference_replay(seq, num_layers):
    """The driver's variables and branches, kept in the driver's order."""
    before_attn, current_attn, before_distance, current_distance, diff = [], [], [], [], []
    transition, at = False, None
    for step, attn_lst in enumerate(seq):
        if transition:
            break
        if len(before_attn) == 0:
            for l in range(num_layers):
                before_attn.append(attn_lst[l]); current_attn.append(attn_lst[l])
        else:
            for l in range(num_layers):
                current_attn[l] = attn_lst[l]
            if len(before_distance) == 0:
                for l in range(num_layers):
                    d = torch.sqrt(torch.sum(torch.pow(before_attn[l] - current_attn[l], 2)))
                    before_distance.append(d); current_distance.append(d); diff.append(0)
            else:
                cnt = 0
                for l in range(num_layers):
                    current_distance[l] = torch.sqrt(torch.sum(torch.pow(before_attn[l] - current_attn[l], 2)))
                    diff[l] = (abs(current_distance[l] - before_distance[l]) / before_distance[l]) * 100
                    before_distance[l] = current_distance[l]
                    if int(diff[l]) < 15:
                        cnt += 1
                if cnt == num_layers:
                    transition, at = True, step + 1
                else:
                    for l in range(num_layers):
                        before_attn[l] = current_attn[l]
    return transition, at


def make_seq(kind, n=8, L=16, layers=2):
    g = torch.Generator().manual_seed(7)
    base = [torch.softmax(torch.randn(L, L, generator=g), -1) for _ in range(layers)]
    seq = []
    for k in range(n):
        if kind == "settling":
            amp = 0.5 * (0.9 ** k) if k < 4 else 0.5 * (0.9 ** 4)
        elif kind == "noisy":
            amp = 0.5 * (2.0 if k % 2 else 0.3)
        else:
            amp = 0.5 / (k + 1)
        seq.append([b + amp * torch.randn(L, L, generator=g) for b in base])
    return seq


def test_matches_driver_replay():
    for kind in ("settling", "noisy", "decay"):
        seq = make_seq(kind)
        det = TransitionDetector(2)
        fired = None
        for k, maps in enumerate(seq):
            if det.update(maps) and fired is None:
                fired = k + 1
        want, at = reference_replay(seq, 2)
        assert det.transition == want and fired == at, kind


def test_needs_three_checks_and_latches():
    maps = [torch.eye(4), torch.eye(4)]
    det = TransitionDetector(2)
    assert det.update(maps) is False
    assert det.update([m + 0.1 for m in maps]) is False
    assert det.update([m + 0.2 for m in maps]) is False     # distance doubled: 100 % change, keep training dense
    assert det.update([m + 0.41 for m in maps]) is True      # distance 0.8 -> 0.84 against the refreshed map: 5 % < 15 %
    assert det.update(maps) is True                          # latched


def test_mask_pickle_round_trip(tmp_path):
    """The mask list travels as the reference pickles it (main_conv_ff.py:298-306): a [4, layers, nb, nb] fp32
    tensor dumped with pickle; a file written the reference's way loads through load_mask_pickle and back."""
    import pickle
    import numpy as np
    import torch
    from oracle import pattern as opat
    from spion_b200 import pattern, synthetic
    mats = [synthetic.band_random_mask(1, 8, 0.3), synthetic.band_random_mask(2, 8, 0.2)]
    mat_lst = torch.as_tensor(opat.stack_for_reference(mats))
    assert mat_lst.shape == (4, 2, 8, 8) and mat_lst.dtype == torch.float32
    ours = tmp_path / "mat_lst_ours.pickle"
    pattern.save_mask_pickle(mat_lst, str(ours))
    with open(ours, "rb") as f:                                   # readable the reference's way (main_inference.py:164-166)
        back = pickle.load(f)
    assert torch.equal(back, mat_lst)
    theirs = tmp_path / "mat_lst_theirs.pickle"
    with open(theirs, "wb") as f:                                 # written the reference's way
        pickle.dump(mat_lst, f, pickle.HIGHEST_PROTOCOL)
    got = pattern.load_mask_pickle(str(theirs))
    assert torch.equal(got, mat_lst)
    for layer in range(2):
        assert np.array_equal(got[0][layer].numpy().astype(np.uint8), mats[layer])
