"""Host-side pieces of the MXFP8 path (plain torch, no GPU): the scale rule, the atom order of the scale words and
the weight quantiser against its dequantiser."""
import pytest
import torch

moe = pytest.importorskip("rbruck_alltoallv_b200.ops.moe")


def test_scale_exponent_is_the_smallest_power_of_two_that_fits():
    amax = torch.tensor([0.0, 1e-3, 1.0, 224.0, 447.9, 448.0, 448.1, 896.0, 1e6])
    e = moe._mx_exponents(amax)
    assert e[0].item() == 0                                   # an all-zero block keeps the scale 1
    nz = amax[1:]
    scaled = nz / torch.exp2(e[1:].float())
    assert torch.all(scaled <= 448.0) and torch.all(scaled > 224.0)   # fits, and one power of two less would not
    assert moe._mx_exponents(torch.tensor([448.0])).item() == 0
    assert moe._mx_exponents(torch.tensor([896.0])).item() == 1


def test_atom_order_is_a_permutation_inside_blocks_of_128_rows():
    n = 300
    plain = torch.arange(2 * n, dtype=torch.int32).view(2, n)
    atoms = moe.mx_to_atoms(plain)
    assert atoms.shape == (2, 384)
    # row r of a block sits at word (r % 32) * 4 + r // 32 of its 128-word atom
    for r in (0, 1, 31, 32, 33, 127, 128, 255, 299):
        pos = (r // 128) * 128 + (r % 32) * 4 + (r % 128) // 32
        assert atoms[0, pos].item() == r and atoms[1, pos].item() == n + r
    assert torch.equal(moe.mx_from_atoms(atoms, n), plain)
    # the padding rows of the last atom carry the scale 1.0 (four bytes of 127)
    used = torch.zeros(384, dtype=torch.bool)
    used[moe._mx_atom_perm(384, "cpu")[:n]] = True
    assert torch.all(atoms[:, ~used] == 0x7f7f7f7f)


def test_weight_quantiser_round_trip_and_scale_packing():
    torch.manual_seed(0)
    G, N, K = 2, 128, 256
    w = torch.randn(G, N, K) * 0.05
    w[0, 3, :32] = 0.0
    w[1, 5, 32:64] *= 1000.0
    q, sf = moe.quantize_weight_mxfp8(w)
    assert q.shape == (G, N, K) and q.dtype == torch.uint8 and sf.shape == (G, K // 128, N) and sf.dtype == torch.int32
    d = moe.dequantize_weight_mxfp8(q, sf)
    blk_max = w.view(G, N, K // 32, 32).abs().amax(dim=3, keepdim=True)
    err = (d - w).view(G, N, K // 32, 32).abs()
    assert torch.all(err <= blk_max / 16 + 1e-12)            # e4m3: 3 mantissa bits under a scale within 2x of amax
    words = moe.mx_from_atoms(sf, N)                           # [G, K/128, N]
    byte = lambda g, n, kblk: (int(words[g, kblk // 4, n].item()) >> (8 * (kblk % 4))) & 0xFF
    assert byte(0, 3, 0) == 127                                # zero block: scale 1
    assert byte(1, 5, 1) > byte(1, 5, 0) + 8                   # the block scaled by 1000 got a scale ~2^10 larger
