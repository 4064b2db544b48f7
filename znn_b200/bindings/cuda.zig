//! Zig declarations of the C ABI of libznn_cuda.so (include/znn_cuda.h), for the host side of chen-gz/znn.
//!
//! UNVERIFIED: written without a Zig toolchain (none was available where this library was built); the prototypes
//! follow the header one to one.  Link with `exe.linkSystemLibrary("znn_cuda")` and add this file as a module.
//! `znn_sgemm` has exactly the prototype of `cblas_sgemm` in src/cblas.zig:17-34, with DEVICE pointers:
//!
//!     pub const cblas_sgemm = switch (backend) {
//!         .accelerate => cblas_sgemm_accelerate,
//!         .cuda => @import("cuda.zig").sgemm_void,     // below: drops the status code like the void prototype
//!         else => cblas_sgemm_fallback,
//!     };
//!
//! Every function returns 0 or a negative ZNN_ERR_* code; `check` turns that into a Zig error.

pub const OK: c_int = 0;
pub const ERR_INVALID: c_int = -1;
pub const ERR_CUDA: c_int = -2;
pub const ERR_NOMEM: c_int = -3;
pub const ERR_DEVICE_WAIT: c_int = -4;
pub const ERR_NCCL: c_int = -5;
pub const ERR_UNSUPPORTED: c_int = -6;

pub const DEV_TMA_WAIT_EXPIRED: c_int = 1;
pub const DEV_MMA_WAIT_EXPIRED: c_int = 2;
pub const DEV_EPI_WAIT_EXPIRED: c_int = 4;
pub const DEV_BAD_INDEX: c_int = 8;

pub const ROW_MAJOR: c_int = 101; // src/cblas.zig:5-8
pub const COL_MAJOR: c_int = 102;
pub const NO_TRANS: c_int = 111;
pub const TRANS: c_int = 112;

pub const TRI_NONE: c_int = 0;
pub const TRI_C_LOWER: c_int = 1;
pub const TRI_A_LOWER: c_int = 2;
pub const TRI_A_UPPER: c_int = 3;
pub const TRI_B_LOWER: c_int = 4;

pub const znn_arena = opaque {};
pub const znn_param_slab = opaque {};

pub const Error = error{ Invalid, Cuda, OutOfDeviceMemory, DeviceWait, Nccl, Unsupported };

pub fn check(rc: c_int) Error!void {
    return switch (rc) {
        0 => {},
        -1 => Error.Invalid,
        -3 => Error.OutOfDeviceMemory,
        -4 => Error.DeviceWait,
        -5 => Error.Nccl,
        -6 => Error.Unsupported,
        else => Error.Cuda,
    };
}

/// cblas_sgemm's void prototype over znn_sgemm (device pointers); a failure is left in znn_last_error and in the
/// device status word, as the reference's own seam has no error channel (src/cblas.zig:17-34).
pub fn sgemm_void(order: c_int, trans_a: c_int, trans_b: c_int, m: c_int, n: c_int, k: c_int, alpha: f32, a: [*]const f32, lda: c_int, b: [*]const f32, ldb: c_int, beta: f32, c: [*]f32, ldc: c_int) callconv(.c) void {
    _ = znn_sgemm(order, trans_a, trans_b, m, n, k, alpha, a, lda, b, ldb, beta, c, ldc);
}

pub extern fn znn_init(device: c_int) c_int;
pub extern fn znn_set_device(device: c_int) c_int;
pub extern fn znn_device_count(count: ?*c_int) c_int;
pub extern fn znn_set_stream(cuda_stream: ?*anyopaque) c_int;
pub extern fn znn_get_stream(cuda_stream: *?*anyopaque) c_int;
pub extern fn znn_sync() c_int;
pub extern fn znn_malloc(ptr: *?*anyopaque, bytes: usize) c_int;
pub extern fn znn_free(ptr: ?*anyopaque) c_int;
pub extern fn znn_memset(ptr: ?*anyopaque, value: c_int, bytes: usize) c_int;
pub extern fn znn_memcpy_h2d(dst: ?*anyopaque, src: ?*const anyopaque, bytes: usize) c_int;
pub extern fn znn_memcpy_d2h(dst: ?*anyopaque, src: ?*const anyopaque, bytes: usize) c_int;
pub extern fn znn_memcpy_d2h_async(dst: ?*anyopaque, src: ?*const anyopaque, bytes: usize) c_int;
pub extern fn znn_memcpy_d2d(dst: ?*anyopaque, src: ?*const anyopaque, bytes: usize) c_int;
pub extern fn znn_memcpy2d_d2d(dst: ?*anyopaque, dst_pitch: usize, src: ?*const anyopaque, src_pitch: usize, width_bytes: usize, rows: usize) c_int;
pub extern fn znn_arena_create(bytes: usize, out: *?*znn_arena) c_int;
pub extern fn znn_arena_alloc(a: ?*znn_arena, bytes: usize, ptr: *?*anyopaque) c_int;
pub extern fn znn_arena_reset(a: ?*znn_arena) c_int;
pub extern fn znn_arena_usage(a: ?*znn_arena, used: ?*usize, high_water: ?*usize, capacity: ?*usize) c_int;
pub extern fn znn_arena_destroy(a: ?*znn_arena) c_int;
pub extern fn znn_param_slab_create(counts: ?[*]const usize, n: c_int, out: *?*znn_param_slab) c_int;
pub extern fn znn_param_slab_total(s: ?*znn_param_slab, total_floats: ?*usize) c_int;
pub extern fn znn_param_slab_tensor(s: ?*znn_param_slab, i: c_int, value: *?[*]f32, grad: *?[*]f32, velocity: *?[*]f32, offset: ?*usize) c_int;
pub extern fn znn_param_slab_zero_grad(s: ?*znn_param_slab) c_int;
pub extern fn znn_param_slab_sgd_step(s: ?*znn_param_slab, lr: f32, momentum: f32, grad_scale: f32) c_int;
pub extern fn znn_param_slab_allreduce_grads(s: ?*znn_param_slab) c_int;
pub extern fn znn_param_slab_destroy(s: ?*znn_param_slab) c_int;
pub extern fn znn_last_error(buf: [*]u8, buflen: usize) c_int;
pub extern fn znn_device_status(status: ?*c_int, clear: c_int) c_int;
pub extern fn znn_gemm_workspace_reserve(bytes: usize) c_int;
pub extern fn znn_launch_count(count: ?*c_longlong, reset: c_int) c_int;
pub extern fn znn_workspace_generation(generation: ?*c_ulonglong) c_int;
pub extern fn znn_sgemm(order: c_int, trans_a: c_int, trans_b: c_int, M: c_int, N: c_int, K: c_int, alpha: f32, A: ?[*]const f32, lda: c_int, B: ?[*]const f32, ldb: c_int, beta: f32, C: ?[*]f32, ldc: c_int) c_int;
pub extern fn znn_sgemm_batched_strided(trans_a: c_int, trans_b: c_int, M: c_int, N: c_int, K: c_int, alpha: f32, A: ?[*]const f32, lda: c_int, stride_a: c_longlong, B: ?[*]const f32, ldb: c_int, stride_b: c_longlong, beta: f32, C: ?[*]f32, ldc: c_int, stride_c: c_longlong, batch: c_int) c_int;
pub extern fn znn_sgemm_host(order: c_int, trans_a: c_int, trans_b: c_int, M: c_int, N: c_int, K: c_int, alpha: f32, A: ?[*]const f32, lda: c_int, B: ?[*]const f32, ldb: c_int, beta: f32, C: ?[*]f32, ldc: c_int, panels: c_int) c_int;
pub extern fn znn_matmul_host_fwd_bwd(A: ?[*]const f32, B: ?[*]const f32, dC: ?[*]const f32, C: ?[*]f32, dA: ?[*]f32, dB: ?[*]f32, M: c_int, K: c_int, N: c_int, accumulate: c_int, panels: c_int) c_int;
pub extern fn znn_sgemm_batched_strided_tri(trans_a: c_int, trans_b: c_int, M: c_int, N: c_int, K: c_int, alpha: f32, A: ?[*]const f32, lda: c_int, stride_a: c_longlong, B: ?[*]const f32, ldb: c_int, stride_b: c_longlong, beta: f32, C: ?[*]f32, ldc: c_int, stride_c: c_longlong, batch: c_int, tri: c_int) c_int;
pub extern fn znn_attn_dscores(dO: ?[*]const f32, V: ?[*]const f32, P: ?[*]const f32, D: ?[*]const f32, scale: f32, dS: ?[*]f32, T: c_int, hs: c_int, nslices: c_int) c_int;
pub extern fn znn_attn_fwd(Q: ?[*]const f32, K: ?[*]const f32, V: ?[*]const f32, O: ?[*]f32, LSE: ?[*]f32, B: c_int, nh: c_int, T: c_int, hs: c_int, ld: c_longlong, stride_h: c_longlong, stride_b: c_longlong, scale: f32) c_int;
pub extern fn znn_attn_bwd(Q: ?[*]const f32, K: ?[*]const f32, V: ?[*]const f32, O: ?[*]const f32, dO: ?[*]const f32, LSE: ?[*]const f32, dQ: ?[*]f32, dK: ?[*]f32, dV: ?[*]f32, B: c_int, nh: c_int, T: c_int, hs: c_int, ld: c_longlong, stride_h: c_longlong, stride_b: c_longlong, scale: f32, accumulate: c_int) c_int;
pub extern fn znn_rowdot(A: ?[*]const f32, B: ?[*]const f32, out: ?[*]f32, rows: usize, D: c_int) c_int;
pub extern fn znn_linear_fwd(X: ?[*]const f32, W: ?[*]const f32, bias: ?[*]const f32, Y: ?[*]f32, M: c_int, K: c_int, N: c_int) c_int;
pub extern fn znn_linear_bwd(X: ?[*]const f32, W: ?[*]const f32, dY: ?[*]const f32, dX: ?[*]f32, dW: ?[*]f32, dbias: ?[*]f32, M: c_int, K: c_int, N: c_int) c_int;
pub extern fn znn_sgemm_grouped(trans_a: c_int, trans_b: c_int, M: c_int, N: c_int, K: c_int, alpha: f32, A: ?[*]const f32, lda: c_int, stride_a: c_longlong, B: ?[*]const f32, ldb: c_int, stride_b: c_longlong, beta: f32, C: ?[*]f32, ldc: c_int, stride_c: c_longlong, batch: c_int, bias: ?[*]const f32, stride_bias: c_longlong, kcat: c_int) c_int;
pub extern fn znn_linear_fwd_ex(X: ?[*]const f32, W: ?[*]const f32, bias: ?[*]const f32, Y: ?[*]f32, pre: ?[*]f32, residual: ?[*]const f32, M: c_int, K: c_int, N: c_int, act: c_int) c_int;
pub extern fn znn_linear_bwd_ex(X: ?[*]const f32, W: ?[*]const f32, dY: ?[*]const f32, dX: ?[*]f32, dW: ?[*]f32, dbias: ?[*]f32, M: c_int, K: c_int, N: c_int, x_pre: ?[*]const f32, x_act: c_int, dx_fresh: c_int) c_int;
pub extern fn znn_gemm_set_path(path: c_int) c_int;
pub extern fn znn_gemm_last_path() c_int;
pub extern fn znn_gemm_set_chunk(k_elements: c_int) c_int;
pub extern fn znn_gemm_set_splitk(enable: c_int) c_int;
pub extern fn znn_add_bias_fwd(A: ?[*]const f32, bias: ?[*]const f32, C: ?[*]f32, M: c_int, N: c_int) c_int;
pub extern fn znn_add_bias_bwd(dC: ?[*]const f32, dA: ?[*]f32, dbias: ?[*]f32, M: c_int, N: c_int) c_int;
pub extern fn znn_relu_fwd(A: ?[*]const f32, C: ?[*]f32, n: usize) c_int;
pub extern fn znn_relu_bwd(A: ?[*]const f32, dC: ?[*]const f32, dA: ?[*]f32, n: usize) c_int;
pub extern fn znn_gelu_fwd(A: ?[*]const f32, C: ?[*]f32, n: usize) c_int;
pub extern fn znn_gelu_bwd(A: ?[*]const f32, dC: ?[*]const f32, dA: ?[*]f32, n: usize) c_int;
pub extern fn znn_gelu_bwd_set(A: ?[*]const f32, dC: ?[*]const f32, dA: ?[*]f32, n: usize) c_int;
pub extern fn znn_softmax_xent_fwd(logits: ?[*]const f32, targets: ?[*]const i32, probs: ?[*]f32, loss: ?[*]f32, M: c_int, N: c_int) c_int;
pub extern fn znn_softmax_xent_fwd_u8(logits: ?[*]const f32, targets: ?[*]const u8, probs: ?[*]f32, loss: ?[*]f32, M: c_int, N: c_int) c_int;
pub extern fn znn_softmax_xent_bwd(probs: ?[*]const f32, targets: ?[*]const i32, dlogits: ?[*]f32, M: c_int, N: c_int) c_int;
pub extern fn znn_softmax_xent_bwd_u8(probs: ?[*]const f32, targets: ?[*]const u8, dlogits: ?[*]f32, M: c_int, N: c_int) c_int;
pub extern fn znn_softmax_xent_fwd_static(logits: ?[*]const f32, targets: ?[*]const i32, probs: ?[*]f32, loss: ?[*]f32, M: c_int, N: c_int, cuda_stream: ?*anyopaque) c_int;
pub extern fn znn_softmax_fwd(A: ?[*]const f32, C: ?[*]f32, rows: usize, D: c_int) c_int;
pub extern fn znn_softmax_bwd(Y: ?[*]const f32, dY: ?[*]const f32, dA: ?[*]f32, rows: usize, D: c_int) c_int;
pub extern fn znn_causal_softmax_fwd(S: ?[*]const f32, scale: f32, P: ?[*]f32, nslices: c_int, T: c_int) c_int;
pub extern fn znn_causal_softmax_bwd(P: ?[*]const f32, dP: ?[*]const f32, scale: f32, dS: ?[*]f32, nslices: c_int, T: c_int) c_int;
pub extern fn znn_causal_softmax_bwd_set(P: ?[*]const f32, dP: ?[*]const f32, scale: f32, dS: ?[*]f32, nslices: c_int, T: c_int) c_int;
pub extern fn znn_rmsnorm_fwd(X: ?[*]const f32, G: ?[*]const f32, eps: f32, Y: ?[*]f32, rows: usize, D: c_int) c_int;
pub extern fn znn_rmsnorm_bwd(X: ?[*]const f32, G: ?[*]const f32, dY: ?[*]const f32, eps: f32, dX: ?[*]f32, dG: ?[*]f32, rows: usize, D: c_int) c_int;
pub extern fn znn_layernorm_fwd(X: ?[*]const f32, G: ?[*]const f32, B: ?[*]const f32, eps: f32, Y: ?[*]f32, rows: usize, D: c_int) c_int;
pub extern fn znn_layernorm_bwd(X: ?[*]const f32, G: ?[*]const f32, dY: ?[*]const f32, eps: f32, dX: ?[*]f32, dG: ?[*]f32, dB: ?[*]f32, rows: usize, D: c_int) c_int;
pub extern fn znn_conv2d_fwd(X: ?[*]const f32, W: ?[*]const f32, bias: ?[*]const f32, Y: ?[*]f32, N: c_int, Ci: c_int, H: c_int, Wd: c_int, Co: c_int, KH: c_int, KW: c_int, pad: c_int) c_int;
pub extern fn znn_conv2d_fwd_act(X: ?[*]const f32, W: ?[*]const f32, bias: ?[*]const f32, Y: ?[*]f32, N: c_int, Ci: c_int, H: c_int, Wd: c_int, Co: c_int, KH: c_int, KW: c_int, pad: c_int, act: c_int) c_int;
pub extern fn znn_conv2d_bwd(X: ?[*]const f32, W: ?[*]const f32, dY: ?[*]const f32, dX: ?[*]f32, dW: ?[*]f32, dbias: ?[*]f32, N: c_int, Ci: c_int, H: c_int, Wd: c_int, Co: c_int, KH: c_int, KW: c_int, pad: c_int) c_int;
pub extern fn znn_maxpool2d_fwd(X: ?[*]const f32, Y: ?[*]f32, idx: ?[*]i32, N: c_int, C: c_int, H: c_int, W: c_int, pool: c_int, stride: c_int) c_int;
pub extern fn znn_maxpool2d_bwd(X: ?[*]const f32, dY: ?[*]const f32, dX: ?[*]f32, N: c_int, C: c_int, H: c_int, W: c_int, pool: c_int, stride: c_int) c_int;
pub extern fn znn_maxpool2d_bwd_relu(X: ?[*]const f32, dY: ?[*]const f32, dX: ?[*]f32, N: c_int, C: c_int, H: c_int, W: c_int, pool: c_int, stride: c_int) c_int;
pub extern fn znn_embedding_fwd(W: ?[*]const f32, ids: ?[*]const f32, Y: ?[*]f32, n: usize, D: c_int, vocab: c_int) c_int;
pub extern fn znn_embedding_bwd(ids: ?[*]const f32, dY: ?[*]const f32, dW: ?[*]f32, n: usize, D: c_int, vocab: c_int) c_int;
pub extern fn znn_transpose_fwd(A: ?[*]const f32, C: ?[*]f32, dims: ?[*]const i64, rank: c_int, d0: c_int, d1: c_int) c_int;
pub extern fn znn_transpose_bwd(dC: ?[*]const f32, dA: ?[*]f32, dims: ?[*]const i64, rank: c_int, d0: c_int, d1: c_int) c_int;
pub extern fn znn_add_fwd(A: ?[*]const f32, B: ?[*]const f32, C: ?[*]f32, n: usize) c_int;
pub extern fn znn_accumulate(src: ?[*]const f32, dst: ?[*]f32, n: usize) c_int;
pub extern fn znn_mul_scalar_fwd(A: ?[*]const f32, v: f32, C: ?[*]f32, n: usize) c_int;
pub extern fn znn_mul_scalar_bwd(dC: ?[*]const f32, v: f32, dA: ?[*]f32, n: usize) c_int;
pub extern fn znn_argmax(A: ?[*]const f32, out: ?[*]f32, M: c_int, N: c_int, dim: c_int) c_int;
pub extern fn znn_accuracy_u8(logits: ?[*]const f32, labels: ?[*]const u8, M: c_int, N: c_int, acc: ?[*]f32) c_int;
pub extern fn znn_sgd_step(w: ?[*]f32, g: ?[*]const f32, v: ?[*]f32, lr: f32, momentum: f32, grad_scale: f32, n: usize) c_int;
pub extern fn znn_adam_step(w: ?[*]f32, g: ?[*]const f32, m: ?[*]f32, v: ?[*]f32, lr: f32, beta1: f32, beta2: f32, eps: f32, t: f32, grad_scale: f32, n: usize) c_int;
pub extern fn znn_pixels_to_unit(pixels: ?[*]const u8, out: ?[*]f32, n: usize) c_int;
pub extern fn znn_batch_gather(images: ?[*]const f32, labels: ?[*]const u8, indices: ?[*]const i32, x_dest: ?[*]f32, y_dest: ?[*]u8, batch: c_int, input_dim: c_int, num_samples: usize) c_int;
pub extern fn znn_fill(dst: ?[*]f32, value: f32, n: usize) c_int;
pub extern fn znn_iota_mod(dst: ?[*]f32, n: usize, period: c_int) c_int;
pub extern fn znn_init_he_normal(w: ?[*]f32, n: usize, fan_in: usize, seed: c_ulonglong) c_int;
pub extern fn znn_fill_normal(w: ?[*]f32, n: usize, mean: f32, stddev: f32, seed: c_ulonglong) c_int;
pub extern fn znn_fill_uniform(w: ?[*]f32, n: usize, min_val: f32, max_val: f32, seed: c_ulonglong) c_int;
pub extern fn znn_dp_unique_id(out128: [*]u8) c_int;
pub extern fn znn_dp_init(world: c_int, rank: c_int, id128: [*:0]const u8) c_int;
pub extern fn znn_dp_init_all(ndev: c_int) c_int;
pub extern fn znn_dp_group_begin() c_int;
pub extern fn znn_dp_group_end() c_int;
pub extern fn znn_dp_world(world: ?*c_int, rank: ?*c_int) c_int;
pub extern fn znn_dp_allreduce_async(buf: ?[*]f32, count: usize) c_int;
pub extern fn znn_dp_join() c_int;
pub extern fn znn_dp_allreduce(buf: ?[*]f32, count: usize) c_int;
pub extern fn znn_dp_broadcast(buf: ?[*]f32, count: usize, root: c_int) c_int;
pub extern fn znn_dp_set_timeout_ms(ms: c_longlong) c_int;
pub extern fn znn_dp_wait(timeout_ms: c_longlong) c_int;
pub extern fn znn_dp_abort() c_int;
pub extern fn znn_dp_finalize() c_int;
