"""sglang-flavoured entry points of part 2: apply_rope_pos_ids_cos_sin_cache (RoPE from an fp32 cos||sin cache, optional
save of the rotated K and of V into token-indexed buffers; op/sglang/csrc/elementwise/rope.cu:28-171) and store_kv_cache
(op/sglang/csrc/memory/store.cu:72-150).  Both run on the kernels of the vLLM-flavoured operators, so the rotated
values are bit-exact against the same oracle; the placement is checked against plain indexing."""
import pytest
import torch

from oracle import ref_ops as R


def _cache(max_pos, rot, base=10000.0):
    inv = 1.0 / (base ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    f = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    return torch.cat([f.cos(), f.sin()], dim=-1)


@pytest.mark.gpu
@pytest.mark.parametrize("n,Hq,Hk,D,rot,interleave,dtype,inplace,save", [
    (77, 8, 2, 128, 128, False, torch.bfloat16, True, False), (77, 8, 2, 128, 128, True, torch.bfloat16, False, True),
    (300, 32, 8, 128, 64, False, torch.float16, True, True), (5000, 16, 4, 64, 64, False, torch.bfloat16, False, True),
    (20000, 32, 8, 128, 128, False, torch.bfloat16, True, True), (3000, 8, 2, 128, 128, False, torch.float16, True, True),
    (9, 4, 4, 256, 128, True, torch.float16, False, False)])
def test_apply_rope_pos_ids_cos_sin_cache(n, Hq, Hk, D, rot, interleave, dtype, inplace, save):
    from mcoplib_b200 import op
    from tests.gpu_util import DEV, bits
    g = torch.Generator().manual_seed(n + Hq)
    q = torch.randn(n, Hq, D, generator=g).to(dtype)
    k = torch.randn(n, Hk, D, generator=g).to(dtype)
    v = torch.randn(n, Hk, D, generator=g).to(dtype)
    pos = torch.randint(0, 4096, (n,), generator=g, dtype=torch.int64)
    cache = _cache(4096, rot)
    q_ref, k_ref = R.rotary_embedding(pos, q.reshape(n, -1), k.reshape(n, -1), D, cache, not interleave)
    qd, kd = q.to(DEV), k.to(DEV)
    q_out = qd if inplace else torch.full_like(qd, 7.0)
    k_out = kd if inplace else torch.full_like(kd, 7.0)
    kw = {}
    if save:
        slots = 2 * n + 3
        loc = torch.randperm(slots, generator=g)[:n].to(torch.int64)
        kbuf = torch.full((slots, Hk, D), 3.0, dtype=dtype, device=DEV)
        vbuf = torch.full((slots, Hk, D), 3.0, dtype=dtype, device=DEV)
        kw = dict(v=v.to(DEV), k_buffer=kbuf, v_buffer=vbuf, kv_cache_loc=loc.to(DEV))
    op.apply_rope_pos_ids_cos_sin_cache(qd, kd, q_out, k_out, cache.to(DEV), pos.to(DEV), interleave, False, **kw)
    assert torch.equal(bits(q_out.cpu().reshape(n, -1)), bits(q_ref)) and torch.equal(bits(k_out.cpu().reshape(n, -1)), bits(k_ref))
    if not inplace:
        assert torch.equal(qd.cpu(), q) and torch.equal(kd.cpu(), k)      # the sources are left alone
    if save:
        kb, vb = kbuf.cpu(), vbuf.cpu()
        assert torch.equal(bits(kb[loc].reshape(n, -1)), bits(k_ref)) and torch.equal(vb[loc], v)
        rest = torch.ones(slots, dtype=torch.bool); rest[loc] = False
        assert bool((kb[rest] == 3.0).all()) and bool((vb[rest] == 3.0).all())


@pytest.mark.gpu
@pytest.mark.parametrize("n", [2500, 64])
def test_apply_rope_save_skips_bad_rows_of_the_buffers(n):
    """The fused rotation + save (one launch from 2048 tokens on; the rotation followed by the copy below that): a negative
    row id rotates the token and stores nothing; a row id past the buffers does the same and records MCOP_DEVERR_SLOT."""
    from mcoplib_b200 import cabi, op
    from tests.gpu_util import DEV, bits
    g = torch.Generator().manual_seed(n)
    Hq, Hk, D = 8, 2, 128
    q = torch.randn(n, Hq, D, generator=g).bfloat16(); k = torch.randn(n, Hk, D, generator=g).bfloat16()
    v = torch.randn(n, Hk, D, generator=g).bfloat16()
    pos = torch.randint(0, 1024, (n,), generator=g, dtype=torch.int64)
    cache = _cache(1024, D)
    q_ref, k_ref = R.rotary_embedding(pos, q.reshape(n, -1), k.reshape(n, -1), D, cache, True)
    slots = n + 10
    loc = torch.randperm(slots, generator=g)[:n].to(torch.int64)
    loc[5] = -1
    loc[7] = slots + 3
    kbuf = torch.full((slots, Hk, D), 3.0, dtype=torch.bfloat16, device=DEV); vbuf = torch.full_like(kbuf, 3.0)
    qd, kd = q.to(DEV), k.to(DEV)
    lib = cabi.load()
    torch.cuda.synchronize(); lib.mcop_device_error()
    op.apply_rope_pos_ids_cos_sin_cache(qd, kd, qd, kd, cache.to(DEV), pos.to(DEV), False, False, v=v.to(DEV), k_buffer=kbuf,
                                        v_buffer=vbuf, kv_cache_loc=loc.to(DEV))
    torch.cuda.synchronize()
    assert lib.mcop_device_error() == cabi.DEVERR_SLOT and lib.mcop_device_error() == 0
    assert torch.equal(bits(qd.cpu().reshape(n, -1)), bits(q_ref)) and torch.equal(bits(kd.cpu().reshape(n, -1)), bits(k_ref))
    good = torch.ones(n, dtype=torch.bool); good[5] = False; good[7] = False
    kb, vb = kbuf.cpu(), vbuf.cpu()
    assert torch.equal(bits(kb[loc[good]].reshape(int(good.sum()), -1)), bits(k_ref[good])) and torch.equal(vb[loc[good]], v[good])
    rest = torch.ones(slots, dtype=torch.bool); rest[loc[good]] = False
    assert bool((kb[rest] == 3.0).all()) and bool((vb[rest] == 3.0).all())


@pytest.mark.gpu
@pytest.mark.parametrize("n,shape,idt,dtype", [(100, (2, 64), torch.int32, torch.bfloat16), (3000, (8, 128), torch.int64, torch.float16),
                                               (17, (1, 512), torch.int64, torch.bfloat16), (64, (64,), torch.int32, torch.float32)])
def test_store_kv_cache(n, shape, idt, dtype):
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    g = torch.Generator().manual_seed(n)
    k = torch.randn(n, *shape, generator=g).to(dtype)
    v = torch.randn(n, *shape, generator=g).to(dtype)
    slots = 3 * n
    loc = torch.randperm(slots, generator=g)[:n].to(idt)
    kc = torch.full((slots, *shape), 5.0, dtype=dtype, device=DEV)
    vc = torch.full((slots, *shape), 5.0, dtype=dtype, device=DEV)
    op.store_kv_cache(kc, vc, loc.to(DEV), k.to(DEV), v.to(DEV))
    assert torch.equal(kc.cpu()[loc.long()], k) and torch.equal(vc.cpu()[loc.long()], v)
    rest = torch.ones(slots, dtype=torch.bool); rest[loc.long()] = False
    assert bool((kc.cpu()[rest] == 5.0).all()) and bool((vc.cpu()[rest] == 5.0).all())


@pytest.mark.gpu
def test_store_kv_cache_rejects_short_rows_and_wrong_index_types():
    from mcoplib_b200 import op
    from tests.gpu_util import DEV
    k = torch.zeros(4, 24, dtype=torch.bfloat16, device=DEV)        # 48 bytes per row
    c = torch.zeros(8, 24, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="divisible by 128"):
        op.store_kv_cache(c, c.clone(), torch.arange(4, device=DEV), k, k.clone())
    k = torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV); c = torch.zeros(8, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(RuntimeError, match="int32 or int64"):
        op.store_kv_cache(c, c.clone(), torch.arange(4, device=DEV).to(torch.int16), k, k.clone())
