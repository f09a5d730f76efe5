"""GPU test of kf_patch_embed_static, the patch embedding for callers that cannot allocate device memory (a plug-in that is
handed inputs and outputs but no allocator; a real-time path that must not call cudaMalloc): its gathered patch rows live
in a fixed array inside the library.  Called through the C-ABI twice in a row, on different images and sizes (the second,
smaller call finds the first call's rows still in the array), it must give the bits of the existing two-call path
(kf_im2col_patch16 into a caller tensor + kf_gemm_bs).  This file is collected last on purpose."""
import pytest
import torch

pytestmark = pytest.mark.gpu
torch.set_grad_enabled(False)
BF = torch.bfloat16


def test_patch_embed_static_matches_the_two_call_path_twice():
    from lightly_trian_quant_b200 import ops
    from lightly_trian_quant_b200._lib import KfError

    g = torch.Generator().manual_seed(5)
    d, npre = 256, 5
    W = ops.QWeight((torch.randn(d, 768, generator=g) * 0.05).cuda(), "bf16")
    bias = (torch.randn(d, generator=g) * 0.1).cuda()
    for B, S in ((2, 160), (1, 96)):                      # 200 rows, then 36: the second call reuses a dirty array
        x = torch.rand(B, 3, S, S, generator=g).to(BF).cuda()
        P = (S // 16) ** 2
        ref = torch.full((B, npre + P, d), -7.0, device="cuda")
        ops.gemm_tokens(ops.im2col_patch16(x), W, bias, ref, P, npre + P, npre)
        out = torch.full((B, npre + P, d), -7.0, device="cuda")
        ops.patch_embed_static(x, W, bias, out, npre)
        ops.check_device_error()
        assert torch.equal(out, ref), (B, S)
        assert torch.isfinite(out[:, npre:]).all() and (out[:, :npre] == -7.0).all()      # rows in front of the patches are not touched
    # beyond the built-in array: refused on the host with a message, nothing launched
    big = torch.zeros(5, 3, 512, 512, dtype=BF, device="cuda")                             # 5 * 1024 rows > 4096
    with pytest.raises(KfError, match="exceed the built-in scratch"):
        ops.patch_embed_static(big, W, bias, torch.empty(5, npre + 1024, d, device="cuda"), npre)
