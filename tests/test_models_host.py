"""Host-side sharding rules of the tensor-parallel linears (no GPU): split_n follows the
reference's largest-remainder cut (src/ucode/ampstein/qwen35_tp.uc:40-72)."""
import pytest

torch = pytest.importorskip("torch")


def test_split_n_equal_weights_largest_remainder():
    from ampstein_b200.models import split_n
    # 25600 columns in 256-units over 8 ranks: 12.5 units each, ties go to the lower ranks
    r = split_n(25600, 256, [1] * 8)
    assert [w for _, w in r] == [3328] * 4 + [3072] * 4
    assert r[0][0] == 0 and all(r[i][0] + r[i][1] == r[i + 1][0] for i in range(7))
    assert r[-1][0] + r[-1][1] == 25600
    assert split_n(14336, 256, [1, 1]) == [(0, 7168), (7168, 7168)]
    # fewer units than ranks: a rank may get nothing
    assert [w for _, w in split_n(512, 256, [1, 1, 1])] == [256, 256, 0]


def test_split_n_weighted():
    from ampstein_b200.models import split_n
    r = split_n(2560, 256, [3, 1])
    assert [w for _, w in r] == [2048, 512] or sum(w for _, w in r) == 2560
    assert sum(w for _, w in r) == 2560


def test_rows_rejects_unaligned_ranges():
    from ampstein_b200.models import LinearEXL3, rows
    lin = LinearEXL3(torch.zeros((16, 8, 64), dtype=torch.int16), torch.ones(256, dtype=torch.float16),
                     torch.ones(128, dtype=torch.float16))
    with pytest.raises(ValueError):
        rows(lin, 64, 128)
    with pytest.raises(ValueError):
        rows(lin, 128, 256)
    part = rows(lin, 128, 128)
    assert part.in_features == 128 and part.out_features == 128 and part.suh.numel() == 128
