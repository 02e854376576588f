"""Host-side mirror of the reference's call surface for the hot path.

Class and method names, argument order and error behaviour follow the reference's C++
classes (Context_23, MLWECiphertext, PCMM_Context, PCMM_Scheme) so that a test written
against this module reads like a reference driver.  Every method forwards to the C ABI
(include/ckks_b200.h); device buffers are torch int64 tensors holding uint64 words
(torch is used for device memory and streams only).
"""
import ctypes as C

import numpy as np
import torch

from . import capi


def _stream_ptr(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def as_u64_tensor(array, device):
    """uint64 numpy array -> int64 device tensor with the same bits."""
    a = np.ascontiguousarray(array, dtype=np.uint64)
    return torch.from_numpy(a.view(np.int64)).to(device)


def to_u64_numpy(tensor):
    return tensor.detach().cpu().contiguous().numpy().view(np.uint64)


class Context_23:
    """Tables and transforms of the reference's Context_23 that lie on the path
    (src/ckks/include/Context_23.h:19-279): moduli [p | q | t], ToNTTInplace,
    FromNTTInplace, modUpQjtoT_23."""

    def __init__(self, logN, pVec, qVec, tVec=(), device=0, gamma=3):
        self.lib = capi.load()
        self.gamma = int(gamma)             # moduli of [p | q] per block of the key-switch chain (Params.cuh:28)
        self.logN, self.N = int(logN), 1 << int(logN)
        self.pVec, self.qVec, self.tVec = list(pVec), list(qVec), list(tVec)
        self.p_num, self.q_num, self.t_num = len(self.pVec), len(self.qVec), len(self.tVec)
        self.K, self.L = self.p_num, self.q_num - 1
        self.device = torch.device("cuda", device)
        self._h = C.c_void_p()
        capi.check(self.lib.ckks_b200_context_create(
            C.byref(self._h), device, self.logN, capi.u64_array(self.pVec), self.p_num,
            capi.u64_array(self.qVec), self.q_num, capi.u64_array(self.tVec), self.t_num))

    def close(self):
        if self._h:
            self.lib.ckks_b200_context_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def psi(self, mod_idx):
        out = C.c_uint64()
        capi.check(self.lib.ckks_b200_context_psi(self._h, mod_idx, C.byref(out)))
        return out.value

    def psi_table(self, mod_idx, inverse=False):
        out = np.zeros(self.N, dtype=np.uint64)
        capi.check(self.lib.ckks_b200_context_table(self._h, mod_idx, int(inverse), out.ctypes.data))
        return out

    # Context_23::ToNTTInplace, src/ckks/include/Context_23.cuh:847-866
    def ToNTTInplace(self, device_a, start_poly_idx, start_mod_idx, poly_num, mod_num, poly_mod_len):
        capi.check(self.lib.ckks_b200_ntt_forward(
            self._h, device_a.data_ptr(), start_poly_idx, start_mod_idx, poly_num, mod_num,
            poly_mod_len, _stream_ptr(self.device)))

    # Context_23::FromNTTInplace, src/ckks/include/Context_23.cuh:868-889
    def FromNTTInplace(self, device_a, start_poly_idx, start_mod_idx, poly_num, mod_num, poly_mod_len):
        capi.check(self.lib.ckks_b200_ntt_inverse(
            self._h, device_a.data_ptr(), start_poly_idx, start_mod_idx, poly_num, mod_num,
            poly_mod_len, _stream_ptr(self.device)))

    # Context_23::modUpQjtoT_23, src/ckks/include/BasisConv.cuh:161-179
    def modUpQjtoT_23(self, output, input, l, batch_size):
        capi.check(self.lib.ckks_b200_modup_qj_to_t(
            self._h, output.data_ptr(), input.data_ptr(), l, batch_size, _stream_ptr(self.device)))

    # ---- key-switch chain (KeySwitch_23.cuh:192-236); gamma is the reference's Context_23::gamma ----
    # Context_23::external_product_T, src/ckks/include/ExternalProduct.cuh:83-97
    def external_product_T(self, output, cipher_modUp_QjtoT, swk_modUp_RitoT, l):
        capi.check(self.lib.ckks_b200_external_product_t(
            self._h, output.data_ptr(), cipher_modUp_QjtoT.data_ptr(), swk_modUp_RitoT.data_ptr(), l, self.gamma,
            _stream_ptr(self.device)))

    # Context_23::FromNTTInplace_for_externalProduct, src/ckks/include/Context_23.cuh:909-930 (as mult_23 calls it)
    def FromNTTInplace_for_externalProduct(self, device_a, l):
        capi.check(self.lib.ckks_b200_ntt_inverse_ext(self._h, device_a.data_ptr(), l, self.gamma, _stream_ptr(self.device)))

    # Context_23::modUpTtoPQl_23, src/ckks/include/BasisConv.cuh:237-248
    def modUpTtoPQl_23(self, modUp_TtoQj_buffer, exProduct_T_temp, l, batch_size):
        capi.check(self.lib.ckks_b200_modup_t_to_pql(
            self._h, modUp_TtoQj_buffer.data_ptr(), exProduct_T_temp.data_ptr(), l, self.gamma, batch_size,
            _stream_ptr(self.device)))

    # Context_23::modDownPQltoQl_23, src/ckks/include/BasisConv.cuh:327-347
    def modDownPQltoQl_23(self, output, modUp_TtoQj_buffer, l, batch_size):
        capi.check(self.lib.ckks_b200_moddown_pql_to_ql(
            self._h, output.data_ptr(), modUp_TtoQj_buffer.data_ptr(), l, self.gamma, batch_size,
            _stream_ptr(self.device)))

    # the chain of Scheme_23::mult_23 between the tensor product and the final addition (:219-232)
    def keyswitch(self, output, input, swk, l):
        capi.check(self.lib.ckks_b200_keyswitch(self._h, output.data_ptr(), input.data_ptr(), swk.data_ptr(), l, self.gamma,
                                                _stream_ptr(self.device)))

    # Kernel choice for modUpQjtoT_23: "auto" (tensor cores where the level's tables qualify),
    # "tensor" (insist) or "simt" (64-bit CUDA-core kernel).  The reference has one kernel.
    def set_modup_algo(self, algo):
        code = {"auto": 0, "tensor": 1, "simt": 2}[algo]
        capi.check(self.lib.ckks_b200_modup_set_algo(self._h, code))

    # Synchronise the current stream; raises on a device-side wait that ran out.
    def check(self):
        capi.check(self.lib.ckks_b200_context_check(self._h, _stream_ptr(self.device)))

    def set_wait_budget(self, cycles):
        """Clock cycles a device-side wait of the tensor-core ModUp may take (0 = the default of about two seconds)."""
        capi.check(self.lib.ckks_b200_context_set_wait_budget(self._h, int(cycles)))

    def test_withhold_commit(self, on=True):
        """Test support: the next tensor-core ModUp leaves out one completion signal so that a wait runs out."""
        capi.check(self.lib.ckks_b200_context_test_withhold_commit(self._h, int(bool(on))))

    def test_exact_count(self, on=True):
        """Test support: every coefficient of a tensor-core ModUp takes the overflow count from IEEE divisions."""
        capi.check(self.lib.ckks_b200_context_test_exact_count(self._h, int(bool(on))))

    # host-buffer forms (numpy uint64 arrays, transformed in place / returned)
    def ToNTTInplace_host(self, host_a, start_poly_idx, start_mod_idx, poly_num, mod_num, poly_mod_len):
        assert host_a.dtype == np.uint64 and host_a.flags.c_contiguous
        capi.check(self.lib.ckks_b200_ntt_forward_host(
            self._h, host_a.ctypes.data, start_poly_idx, start_mod_idx, poly_num, mod_num, poly_mod_len))

    def FromNTTInplace_host(self, host_a, start_poly_idx, start_mod_idx, poly_num, mod_num, poly_mod_len):
        assert host_a.dtype == np.uint64 and host_a.flags.c_contiguous
        capi.check(self.lib.ckks_b200_ntt_inverse_host(
            self._h, host_a.ctypes.data, start_poly_idx, start_mod_idx, poly_num, mod_num, poly_mod_len))

    def modUpQjtoT_23_host(self, host_in, l, batch_size):
        assert host_in.dtype == np.uint64 and host_in.flags.c_contiguous
        blocks = (l + 1 + self.p_num - 1) // self.p_num
        out = np.zeros((batch_size, blocks, self.t_num, self.N), dtype=np.uint64)
        capi.check(self.lib.ckks_b200_modup_qj_to_t_host(
            self._h, out.ctypes.data, host_in.ctypes.data, l, batch_size))
        return out


class Ciphertext:
    """RLWE ciphertext buffer: a limbs then b limbs, each [L+1][N] words, NTT domain at rest
    (src/ckks/include/Ciphertext.cuh:5-100)."""

    def __init__(self, N, L, l, slots, scale, device=0, cipher=None):
        self.N, self.L, self.l, self.slots, self.scale = N, L, l, slots, scale
        if cipher is None:
            cipher = torch.zeros(2 * (L + 1) * N, dtype=torch.int64, device=torch.device("cuda", device))
        self.cipher_device = cipher


class Scheme_23:
    """The level-lowering step of the reference's evaluator that the PCMM pipeline uses
    (src/ckks/include/Scheme_23.cuh:368-385)."""

    def __init__(self, context):
        self.context = context
        self.rotKey_vec_23 = {}

    # Scheme_23::mult_23(cipher_res, cipher1, cipher2), src/ckks/include/KeySwitch_23.cuh:192-236.  rlk_23 is the
    # relinearisation key block [2][dnum][R][t_num][N] (key generation is the caller's).
    rlk_23 = None

    def mult_23(self, cipher_res, cipher1, cipher2):
        if cipher1.l == 0 or cipher2.l == 0:
            raise ValueError("Ciphertexts are on level 0")                 # invalid_argument at :194-197
        if self.rlk_23 is None:
            raise ValueError("rotKey_23 not exists")                       # :198-201
        ctx = self.context
        l = min(cipher1.l, cipher2.l)
        capi.check(ctx.lib.ckks_b200_mult(ctx._h, cipher_res.cipher_device.data_ptr(), cipher1.cipher_device.data_ptr(),
                                          cipher2.cipher_device.data_ptr(), self.rlk_23.data_ptr(), l, ctx.gamma,
                                          _stream_ptr(ctx.device)))
        cipher_res.l = l
        cipher_res.scale = cipher1.scale * cipher2.scale

    # Scheme_23::conjugate_23(cipher_res, cipher) and conjugateAndEqual_23, src/ckks/include/KeySwitch_23.cuh:433-507.
    # ConjKey_23 is the conjugation key block, laid out like rlk_23.
    ConjKey_23 = None

    def conjugate_23(self, cipher_res, cipher):
        if self.ConjKey_23 is None:
            raise ValueError("conjKey_23 not exists")                      # :435-438
        ctx = self.context
        capi.check(ctx.lib.ckks_b200_conjugate(ctx._h, cipher_res.cipher_device.data_ptr(), cipher.cipher_device.data_ptr(),
                                               self.ConjKey_23.data_ptr(), cipher.l, ctx.gamma, _stream_ptr(ctx.device)))
        cipher_res.l = cipher.l
        cipher_res.scale = cipher.scale

    def conjugateAndEqual_23(self, cipher):
        self.conjugate_23(cipher, cipher)

    # Scheme_23::leftRotate_23(cipher_res, cipher, rotSlots) and leftRotateAndEqual_23, KeySwitch_23.cuh:509-581.
    # rotKey_vec_23 maps a rotation to its key block (addLeftRotKey_23 of the reference fills it; key generation is
    # the caller's here).
    def leftRotate_23(self, cipher_res, cipher, rotSlots):
        key = self.rotKey_vec_23.get(rotSlots)
        if key is None:
            raise ValueError("rotKey_23 not exists")                       # :511-514
        ctx = self.context
        capi.check(ctx.lib.ckks_b200_rotate(ctx._h, cipher_res.cipher_device.data_ptr(), cipher.cipher_device.data_ptr(),
                                            key.data_ptr(), int(rotSlots), cipher.l, ctx.gamma, _stream_ptr(ctx.device)))
        cipher_res.l = cipher.l
        cipher_res.scale = cipher.scale

    def leftRotateAndEqual_23(self, cipher, rotSlots):
        self.leftRotate_23(cipher, cipher, rotSlots)

    # Scheme_23::rescaleAndEqual(Ciphertext&), src/ckks/include/Scheme_23.cuh:368-385
    def rescaleAndEqual(self, cipher):
        ctx = self.context
        capi.check(ctx.lib.ckks_b200_rescale(ctx._h, cipher.cipher_device.data_ptr(), cipher.L, cipher.l,
                                             _stream_ptr(ctx.device)))
        cipher.scale = cipher.scale / ctx.qVec[cipher.l]
        cipher.l -= 1

    def rescaleAndEqual_batch(self, ciphers):
        """rescaleAndEqual of several ciphertexts in one pass.  They must be views, in order, of one contiguous device
        buffer (ciphertext i at offset i * 2 * (L+1) * N words) and share L and l."""
        ctx, first = self.context, ciphers[0]
        words = 2 * (first.L + 1) * ctx.N
        base = first.cipher_device.data_ptr()
        for i, c in enumerate(ciphers):
            if c.cipher_device.data_ptr() != base + 8 * i * words or (c.L, c.l) != (first.L, first.l):
                raise ValueError("the batched form needs equally shaped ciphertexts stored one after another")
        capi.check(ctx.lib.ckks_b200_rescale_batch(ctx._h, base, len(ciphers), first.L, first.l, _stream_ptr(ctx.device)))
        for c in ciphers:
            c.scale = c.scale / ctx.qVec[c.l]
            c.l -= 1


class Bootstrapper:
    """The level-raising step in front of the bootstrapping pipeline
    (src/ckks/include/bootstrapping/Bootstrapper.cuh:192-209)."""

    def __init__(self, context, precision):
        self.context = context
        self.precision = int(precision)

    # Bootstrapper::modUpQ0toQL(Ciphertext&, int target_level): a no-op unless the ciphertext is at level 0 (:194)
    def modUpQ0toQL(self, cipher, target_level):
        if cipher.l != 0:
            return
        ctx = self.context
        scale_up = C.c_int(ctx.qVec[0] // self.precision).value      # the kernel's parameter is an int (:6)
        capi.check(ctx.lib.ckks_b200_modup_q0_to_ql(ctx._h, cipher.cipher_device.data_ptr(), cipher.L, target_level,
                                                    scale_up, _stream_ptr(ctx.device)))
        cipher.l = target_level

    def modUpQ0toQL_batch(self, ciphers, target_level):
        """modUpQ0toQL of several level-0 ciphertexts in one pass; the same layout rule as Scheme_23.rescaleAndEqual_batch."""
        ctx, first = self.context, ciphers[0]
        words = 2 * (first.L + 1) * ctx.N
        base = first.cipher_device.data_ptr()
        for i, c in enumerate(ciphers):
            if c.cipher_device.data_ptr() != base + 8 * i * words or c.L != first.L or c.l != 0:
                raise ValueError("the batched form needs level-0 ciphertexts of one shape stored one after another")
        scale_up = C.c_int(ctx.qVec[0] // self.precision).value
        capi.check(ctx.lib.ckks_b200_modup_q0_to_ql_batch(ctx._h, base, len(ciphers), first.L, target_level, scale_up,
                                                          _stream_ptr(ctx.device)))
        for c in ciphers:
            c.l = target_level


class MLWECiphertext:
    """Device buffer [L+1][k+1][N1] words (src/ckks/include/pcmm/MLWECiphertext.cuh:6-78)."""

    def __init__(self, N1, L, l, k, scale, device=0, cipher=None):
        self.N1, self.L, self.l, self.k, self.scale = N1, L, l, k, scale
        if cipher is None:
            cipher = torch.zeros((L + 1) * (k + 1) * N1, dtype=torch.int64, device=torch.device("cuda", device))
        self.cipher_device = cipher


class PCMM_Context:
    """Parameter carrier of the ring packing (src/ckks/include/pcmm/PCMM_Context.h:14-90)."""

    def __init__(self, N1, mlwe_rank, p_ringpack, q_ringpack, device=0):
        self.lib = capi.load()
        self.N1, self.mlwe_rank = int(N1), int(mlwe_rank)
        self.p_ringpack, self.q_ringpack = list(p_ringpack), list(q_ringpack)
        self.ringpack_p_count = len(self.p_ringpack)
        self.ringpack_q_count = len(self.q_ringpack)
        self.ringpack_pq_count = self.ringpack_p_count + self.ringpack_q_count
        self.device = torch.device("cuda", device)
        self._h = C.c_void_p()
        capi.check(self.lib.ckks_b200_pcmm_create(
            C.byref(self._h), device, self.N1, self.mlwe_rank, capi.u64_array(self.q_ringpack),
            self.ringpack_q_count))

    def set_peer_outputs(self, peer_pointers):
        """Device addresses, valid on this GPU, of the other GPUs' output buffers (same layout as the local output)
        that every tensor-core multiply from now on also writes; an empty list switches it off."""
        ptrs = (C.c_void_p * max(len(peer_pointers), 1))(*[int(p) for p in peer_pointers])
        capi.check(self.lib.ckks_b200_pcmm_set_peer_outputs(self._h, ptrs, len(peer_pointers)))

    def set_row_owners(self, out_by_rank, self_rank):
        """Device addresses, valid on this GPU, of every rank's output buffer (the entry of self_rank is ignored): from now
        on a tensor-core multiply stores each output row into its owner's buffer only.  An empty list switches it off."""
        world = len(out_by_rank)
        ptrs = (C.c_void_p * max(world, 1))(*[int(p) if p else None for p in out_by_rank])
        capi.check(self.lib.ckks_b200_pcmm_set_row_owners(self._h, ptrs, world, int(self_rank)))

    def row_owner_range(self, mat_M, world, rank):
        """Rows [begin, end) of a mat_M-row output that belong to `rank` of `world` under set_row_owners."""
        b, e = C.c_int(), C.c_int()
        capi.check(self.lib.ckks_b200_pcmm_row_owner_range(int(mat_M), int(world), int(rank), C.byref(b), C.byref(e)))
        return b.value, e.value

    def set_wait_budget(self, cycles):
        """Clock cycles a device-side wait of the tensor-core multiply may take (0 = the default of about two seconds)."""
        capi.check(self.lib.ckks_b200_pcmm_set_wait_budget(self._h, int(cycles)))

    def test_withhold_stage(self, stage):
        """Test support: the next tensor-core multiply stops feeding operand tiles before tile `stage` of every CTA."""
        capi.check(self.lib.ckks_b200_pcmm_test_withhold_stage(self._h, int(stage)))

    def set_host_chunks(self, chunks):
        """Number of column chunks the host-buffer multiply pipelines through its copy and compute streams (0 = automatic)."""
        capi.check(self.lib.ckks_b200_pcmm_set_host_chunks(self._h, int(chunks)))

    def close(self):
        if self._h:
            self.lib.ckks_b200_pcmm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def ppmm_scaler(q_ringpack, scale, target_scale=float(1 << 49)):
    """scaler = (long)(q_last * target / scale): PPMM_kernel.cuh:283-284 writes q_ringpack[1], the last of the reference's
    two moduli and the one its kernel rescales by; with more limbs that is the last one."""
    return float(int(q_ringpack[-1] * target_scale / scale))


def ppmm_scale_after(q_ringpack, scale, scaler):
    """The scale PPMM leaves on its ciphertexts (PPMM_kernel.cuh:346)."""
    return scale * scaler / q_ringpack[-1]


class PCMM_Scheme:
    """PPMM of the reference's PCMM_Scheme (src/ckks/include/pcmm/PCMM_Scheme.h:12-48)."""

    def __init__(self, pcmm_context, algo=capi.PCMM_AUTO, context=None):
        self.pcmm_context = pcmm_context
        self.context = context              # Context_23, needed by rlweCipherDecompose
        self.lib = pcmm_context.lib
        self.algo = algo
        self.ppmm_output = None

    def scaler_for(self, scale, target_scale=float(1 << 49)):
        """scaler = (long)(q_last * target / scale): PPMM_kernel.cuh:283-284 writes q_ringpack[1], the last of the
        reference's two moduli and the one its kernel rescales by; with more limbs that is the last one."""
        return ppmm_scaler(self.pcmm_context.q_ringpack, scale, target_scale)

    def prepare_weights(self, plain_mat, mat_M, mat_N, scaler):
        """Scale and slice a weight matrix once (ckks_b200_pcmm_prepare_weights); PPMM / decomposeAndPPMM calls that pass
        plain_mat=None with the same shape and scaler then multiply by it without a per-call weight pre-pass."""
        pc = self.pcmm_context
        capi.check(self.lib.ckks_b200_pcmm_prepare_weights(pc._h, plain_mat.data_ptr(), mat_M, mat_N, float(scaler),
                                                           _stream_ptr(pc.device)))

    def PPMM(self, plain_mat, mlwe_cipher_decomposed, mat_M, mat_N, mat_K, mlwe_num, scaler=None,
             col_begin=0, col_end=None, copy_back=True):
        """PCMM_Scheme::PPMM (src/ckks/include/pcmm/PPMM_kernel.cuh:254-349).

        plain_mat: fp32 device tensor [mat_M][mat_N].  Like the reference, a shape
        violation prints its message and returns without computing.  `scaler` defaults to
        the reference's choice.  The raw result stays in self.ppmm_output
        ([mat_M][q_count][(k+1)*N1]); with copy_back the first limb of row i overwrites
        ciphertext i and scales are updated as at :345-348."""
        pc = self.pcmm_context
        if scaler is None:
            scaler = self.scaler_for(mlwe_cipher_decomposed[0].scale)
        C_ = (pc.mlwe_rank + 1) * pc.N1
        if col_end is None:
            col_end = C_
        need = mat_M * pc.ringpack_q_count * C_
        if self.ppmm_output is None or self.ppmm_output.numel() < need:
            self.ppmm_output = torch.empty(need, dtype=torch.int64, device=pc.device)
        ptrs = (C.c_void_p * max(mlwe_num, 1))(*[c.cipher_device.data_ptr() for c in mlwe_cipher_decomposed[:mlwe_num]])
        st = self.lib.ckks_b200_pcmm_ppmm(
            pc._h, plain_mat.data_ptr() if plain_mat is not None else None, ptrs, self.ppmm_output.data_ptr(), mat_M, mat_N,
            mat_K, mlwe_num, float(scaler), col_begin, col_end, self.algo, _stream_ptr(pc.device))
        if st == capi.ERR_SHAPE:
            print(self.lib.ckks_b200_last_error().decode())
            return None
        capi.check(st)
        out = self.ppmm_output[:need].view(mat_M, pc.ringpack_q_count, C_)
        if copy_back:
            capi.check(self.lib.ckks_b200_pcmm_copy_back(
                pc._h, self.ppmm_output.data_ptr(), ptrs, min(mlwe_num, mat_M), 1, _stream_ptr(pc.device)))
            for c in mlwe_cipher_decomposed[:mlwe_num]:
                c.scale = ppmm_scale_after(pc.q_ringpack, c.scale, scaler)
        return out

    def rlweCipherDecompose(self, rlwe_cipher, mlwe_cipher_decomposed, mlwe_num, offset, ntt_domain=True):
        """PCMM_Scheme::rlweCipherDecompose (src/ckks/include/pcmm/PCMM_Scheme.cuh:90-125): fills
        mlwe_cipher_decomposed[offset : offset+mlwe_num] from the RLWE ciphertext.  Like the
        reference, asking for more ciphertexts than the rank prints a message and returns."""
        pc, ctx = self.pcmm_context, self.context
        ptrs = (C.c_void_p * max(mlwe_num, 1))(
            *[c.cipher_device.data_ptr() for c in mlwe_cipher_decomposed[offset:offset + mlwe_num]])
        st = self.lib.ckks_b200_rlwe_decompose(ctx._h, rlwe_cipher.cipher_device.data_ptr(), rlwe_cipher.L, rlwe_cipher.l,
                                               ptrs, mlwe_num, pc.N1, pc.mlwe_rank, int(ntt_domain), _stream_ptr(pc.device))
        if st == capi.ERR_SHAPE:
            print(self.lib.ckks_b200_last_error().decode())
            return
        capi.check(st)

    def decomposeAndPPMM(self, plain_mat, sources, mlwe_cipher_decomposed, mat_M, mat_N, mat_K, mlwe_num, scaler=None,
                         col_begin=0, col_end=None, ntt_domain=True, copy_back=True):
        """rlweCipherDecompose of every (rlwe_cipher, mlwe_num, offset) in `sources` followed by PPMM, as one call
        that never writes the decomposed ciphertexts (PCMM_Scheme.cuh:90-125 feeding PPMM_kernel.cuh:254-349; the
        pairing of calls is Bert.cuh:249-254).  The result is that of the two separate calls, word for word.
        mlwe_cipher_decomposed only receives the copy-back of the result rows, as after PPMM."""
        pc, ctx = self.pcmm_context, self.context
        if scaler is None:
            scaler = self.scaler_for(sources[0][0].scale)
        C_ = (pc.mlwe_rank + 1) * pc.N1
        if col_end is None:
            col_end = C_
        need = mat_M * pc.ringpack_q_count * C_
        if self.ppmm_output is None or self.ppmm_output.numel() < need:
            self.ppmm_output = torch.empty(need, dtype=torch.int64, device=pc.device)
        st_ptr = _stream_ptr(pc.device)
        arr = (capi.RlweSource * max(len(sources), 1))()
        for k, (ct, num, off) in enumerate(sources):
            arr[k].d_rlwe, arr[k].L, arr[k].mlwe_num, arr[k].offset = ct.cipher_device.data_ptr(), ct.L, num, off
        if ntt_domain:
            for ct, _, _ in sources:
                capi.check(self.lib.ckks_b200_ntt_inverse(ctx._h, ct.cipher_device.data_ptr(), 0, ctx.p_num, 2, ct.l + 1,
                                                          ct.L + 1, st_ptr))
        st = self.lib.ckks_b200_pcmm_ppmm_rlwe(pc._h, plain_mat.data_ptr() if plain_mat is not None else None, arr,
                                               len(sources), self.ppmm_output.data_ptr(),
                                               mat_M, mat_N, mat_K, mlwe_num, float(scaler), col_begin, col_end, st_ptr)
        if ntt_domain:
            for ct, _, _ in sources:
                capi.check(self.lib.ckks_b200_ntt_forward(ctx._h, ct.cipher_device.data_ptr(), 0, ctx.p_num, 2, ct.l + 1,
                                                          ct.L + 1, st_ptr))
        if st == capi.ERR_SHAPE:
            print(self.lib.ckks_b200_last_error().decode())
            return None
        capi.check(st)
        out = self.ppmm_output[:need].view(mat_M, pc.ringpack_q_count, C_)
        if copy_back:
            ptrs = (C.c_void_p * max(mlwe_num, 1))(*[c.cipher_device.data_ptr() for c in mlwe_cipher_decomposed[:mlwe_num]])
            capi.check(self.lib.ckks_b200_pcmm_copy_back(pc._h, self.ppmm_output.data_ptr(), ptrs, min(mlwe_num, mat_M), 1, st_ptr))
            for c in mlwe_cipher_decomposed[:mlwe_num]:
                c.scale = ppmm_scale_after(pc.q_ringpack, sources[0][0].scale, scaler)
        return out

    def addRepakcingKey(self, keys_device):
        """The reference generates the keys itself (PCMM_Scheme.cuh:152-223); key generation is
        out of scope here, so the caller hands over the finished block [k][2][2][N]."""
        self.repackingKeys = keys_device

    def mlweCipherPacking(self, rlwe_cipher, mlwe_cipher_decomposed, mlwe_num, offset):
        """PCMM_Scheme::mlweCipherPacking (src/ckks/include/pcmm/PCMM_Scheme.cuh:362-430)."""
        pc, ctx = self.pcmm_context, self.context
        ptrs = (C.c_void_p * max(mlwe_num, 1))(
            *[c.cipher_device.data_ptr() for c in mlwe_cipher_decomposed[offset:offset + mlwe_num]])
        capi.check(self.lib.ckks_b200_mlwe_packing(ctx._h, rlwe_cipher.cipher_device.data_ptr(), rlwe_cipher.L, ptrs,
                                                   mlwe_num, pc.N1, pc.mlwe_rank, self.repackingKeys.data_ptr(),
                                                   _stream_ptr(pc.device)))
        rlwe_cipher.l = pc.ringpack_q_count - 1 - 1                      # :418-420
        rlwe_cipher.scale = mlwe_cipher_decomposed[0].scale

    def check(self):
        capi.check(self.lib.ckks_b200_pcmm_check(self.pcmm_context._h, _stream_ptr(self.pcmm_context.device)))

    def last_timing(self):
        """(pre-pass ms, main kernel ms) of the latest tensor-core multiply."""
        a, b = C.c_float(), C.c_float()
        capi.check(self.lib.ckks_b200_pcmm_last_timing(self.pcmm_context._h, C.byref(a), C.byref(b)))
        return a.value, b.value

    def PPMM_host(self, plain_mat, X, mat_M, mat_N, mat_K, mlwe_num, scaler):
        """Host-buffer call: numpy in, numpy out, copies inside."""
        pc = self.pcmm_context
        W = np.ascontiguousarray(plain_mat, dtype=np.float32)
        X = np.ascontiguousarray(X, dtype=np.uint64)
        C_ = (pc.mlwe_rank + 1) * pc.N1
        out = np.empty((mat_M, pc.ringpack_q_count, C_), dtype=np.uint64)
        capi.check(self.lib.ckks_b200_pcmm_ppmm_host(
            pc._h, W.ctypes.data, X.ctypes.data, out.ctypes.data, mat_M, mat_N, mat_K, mlwe_num,
            float(scaler), self.algo))
        return out

    def PPMM_rlwe_host(self, plain_mat, sources, mat_M, mat_N, mat_K, mlwe_num, scaler, out=None):
        """Host-buffer form of decomposeAndPPMM: `sources` is a list of (rlwe, L, mlwe_num, offset) with rlwe a contiguous
        uint64 array [2][L+1][N] in the coefficient domain; returns the output [mat_M][q_count][(k+1)*N1] (numpy, or the
        given `out`)."""
        pc = self.pcmm_context
        W = np.ascontiguousarray(plain_mat, dtype=np.float32)
        C_ = (pc.mlwe_rank + 1) * pc.N1
        if out is None:
            out = np.empty((mat_M, pc.ringpack_q_count, C_), dtype=np.uint64)
        arr = (capi.RlweSource * max(len(sources), 1))()
        keep = []
        for k, (rl, L, num, off) in enumerate(sources):
            rl = np.ascontiguousarray(rl, dtype=np.uint64)
            keep.append(rl)
            arr[k].d_rlwe, arr[k].L, arr[k].mlwe_num, arr[k].offset = rl.ctypes.data, L, num, off
        capi.check(self.lib.ckks_b200_pcmm_ppmm_rlwe_host(pc._h, W.ctypes.data, arr, len(sources), out.ctypes.data, mat_M,
                                                          mat_N, mat_K, mlwe_num, float(scaler)))
        return out
