# Crystal binding of libshainet_attn.so (C ABI: include/shainet_attn.h).
#
# Link-time binding (no dlopen): build with
#   crystal build -Denable_cuda --link-flags "-L<dir of libshainet_attn.so> -lshainet_attn" ...
# This file is what a SHAInet maintainer would add under src/shainet/; it has
# not been compiled here (no Crystal compiler on the build image).
module SHAInet
  @[Link("shainet_attn")]
  lib LibShainetAttn
    type Ctx = Void*
    type Kv = Void*

    fun version = shainet_attn_version : Int32
    fun device_count = shainet_attn_device_count : Int32
    fun last_error = shainet_attn_last_error : UInt8*

    fun ctx_create = shainet_attn_ctx_create(out_ctx : Ctx*, device : Int32) : Int32
    fun ctx_destroy = shainet_attn_ctx_destroy(ctx : Ctx) : Int32
    fun ctx_sync = shainet_attn_ctx_sync(ctx : Ctx) : Int32

    fun kv_create = shainet_attn_kv_create(ctx : Ctx, out_kv : Kv*, num_heads : Int32, num_kv_heads : Int32,
                                           head_dim : Int32, initial_capacity : Int32) : Int32
    KV_F32  = 0
    KV_BF16 = 1
    fun kv_create_fmt = shainet_attn_kv_create_fmt(ctx : Ctx, out_kv : Kv*, num_heads : Int32, num_kv_heads : Int32,
                                                   head_dim : Int32, initial_capacity : Int32, format : Int32) : Int32
    fun kv_format = shainet_attn_kv_format(kv : Kv) : Int32
    fun kv_create_reserved = shainet_attn_kv_create_reserved(ctx : Ctx, out_kv : Kv*, num_heads : Int32, num_kv_heads : Int32,
                                                             head_dim : Int32, max_capacity : Int32, format : Int32) : Int32
    fun kv_destroy = shainet_attn_kv_destroy(kv : Kv) : Int32
    fun kv_reset = shainet_attn_kv_reset(kv : Kv) : Int32
    fun kv_truncate = shainet_attn_kv_truncate(kv : Kv, len : Int32) : Int32
    fun kv_len = shainet_attn_kv_len(kv : Kv) : Int32
    fun kv_capacity = shainet_attn_kv_capacity(kv : Kv) : Int32
    fun kv_reserve = shainet_attn_kv_reserve(kv : Kv, total_len : Int32) : Int32
    fun kv_set_rope_theta = shainet_attn_kv_set_rope_theta(kv : Kv, theta : Float64) : Int32
    fun kv_set_rope = shainet_attn_kv_set_rope(kv : Kv, inv_freq : Float32*, half : Int32) : Int32
    fun kv_set_qk_norm = shainet_attn_kv_set_qk_norm(kv : Kv, q_w : Float32*, k_w : Float32*, eps : Float64) : Int32
    fun kv_set_bias = shainet_attn_kv_set_bias(kv : Kv, b_q : Float32*, b_k : Float32*, b_v : Float32*) : Int32
    fun kv_export = shainet_attn_kv_export(kv : Kv, k : Float32*, v : Float32*, len : Int32) : Int32
    fun kv_import = shainet_attn_kv_import(kv : Kv, k : Float32*, v : Float32*, len : Int32) : Int32

    fun forward_host = shainet_attn_forward_host(ctx : Ctx, kv : Kv, q : Float32*, k_new : Float32*, v_new : Float32*,
                                                 out_ptr : Float32*, new_tokens : Int32, scale : Float32,
                                                 flags : UInt32) : Int32
    fun forward_dev = shainet_attn_forward_dev(ctx : Ctx, kv : Kv, q : Float32*, k_new : Float32*, v_new : Float32*,
                                               out_ptr : Float32*, new_tokens : Int32, scale : Float32, flags : UInt32,
                                               stream : Void*) : Int32
    fun forward_batched_dev = shainet_attn_forward_batched_dev(ctx : Ctx, kvs : Kv*, batch : Int32, q : Float32*,
                                                               k_new : Float32*, v_new : Float32*, out_ptr : Float32*,
                                                               scale : Float32, flags : UInt32, stream : Void*) : Int32

    # measurement and bookkeeping
    fun ctx_scratch_bytes = shainet_attn_ctx_scratch_bytes(ctx : Ctx) : LibC::SizeT
    fun ctx_timing_enable = shainet_attn_ctx_timing_enable(ctx : Ctx, enable : Int32) : Int32
    fun ctx_timing_read = shainet_attn_ctx_timing_read(ctx : Ctx, total_ms : Float64*, launches : Int32*) : Int32
    fun kv_fill_normal = shainet_attn_kv_fill_normal(kv : Kv, len : Int32, seed : UInt64) : Int32
    fun kv_device_ptrs = shainet_attn_kv_device_ptrs(kv : Kv, k_dev : Float32**, v_dev : Float32**) : Int32

    # a block sharded over the GPUs of one box (one process per GPU)
    fun ctx_set_lse_out = shainet_attn_ctx_set_lse_out(ctx : Ctx, lse_dev : Float32*) : Int32
    fun forward_dev_at = shainet_attn_forward_dev_at(ctx : Ctx, kv : Kv, q : Float32*, k_new : Float32*, v_new : Float32*,
                                                     out_ptr : Float32*, position : Int32, append : Int32, scale : Float32,
                                                     flags : UInt32, stream : Void*) : Int32
    fun merge_parts = shainet_attn_merge_parts(ctx : Ctx, gathered_dev : Float32*, world : Int32, seq_parts : Int32,
                                               heads_per_rank : Int32, head_dim : Int32, out_full_dev : Float32*,
                                               stream : Void*) : Int32
    fun comm_create = shainet_attn_comm_create(ctx : Ctx, data_floats : LibC::SizeT, handle_out : Void*) : Int32
    fun comm_open = shainet_attn_comm_open(ctx : Ctx, handles : Void*, world : Int32, rank : Int32) : Int32
    fun comm_set_target = shainet_attn_comm_set_target(ctx : Ctx, out_offset_floats : Int64, lse_offset_floats : Int64,
                                                       epoch : UInt32) : Int32
    fun comm_wait = shainet_attn_comm_wait(ctx : Ctx, offset_floats : Int64, count_floats : Int64, epoch : UInt32,
                                           stream : Void*) : Int32
    fun forward_dev_exchange = shainet_attn_forward_dev_exchange(ctx : Ctx, kv : Kv, q : Float32*, k_new : Float32*,
                                                                 v_new : Float32*, out_ptr : Float32*, position : Int32,
                                                                 append : Int32, scale : Float32, flags : UInt32,
                                                                 out_offset_floats : Int64, lse_offset_floats : Int64,
                                                                 wait_offset_floats : Int64, wait_count_floats : Int64,
                                                                 epoch : UInt32, stream : Void*) : Int32
    fun forward_dev_exchange_merge = shainet_attn_forward_dev_exchange_merge(ctx : Ctx, kv : Kv, q : Float32*,
                                                                             k_new : Float32*, v_new : Float32*,
                                                                             out_ptr : Float32*, position : Int32,
                                                                             append : Int32, scale : Float32, flags : UInt32,
                                                                             slot_offset_floats : Int64, seq_parts : Int32,
                                                                             epoch : UInt32, out_full_dev : Float32*,
                                                                             stream : Void*) : Int32
    fun comm_set_wait_limit_ms = shainet_attn_comm_set_wait_limit_ms(ctx : Ctx, milliseconds : Int32) : Int32
    fun comm_read = shainet_attn_comm_read(ctx : Ctx, offset_floats : Int64, host_dst : Float32*, floats : LibC::SizeT,
                                           stream : Void*) : Int32
    fun comm_data_ptr = shainet_attn_comm_data_ptr(ctx : Ctx, data_dev : Float32**) : Int32

    # Q8_0 weights, the whole block and the token loop on the device
    type Q8 = Void*
    type Block = Void*
    type Decoder = Void*
    fun q8_create = shainet_attn_q8_create(ctx : Ctx, out_w : Q8*, w_host : Float32*, k : Int32, n : Int32) : Int32
    fun q8_create_raw = shainet_attn_q8_create_raw(ctx : Ctx, out_w : Q8*, q_host : Int8*, scales_host : Float32*,
                                                   k : Int32, n : Int32) : Int32
    fun q8_wrap = shainet_attn_q8_wrap(ctx : Ctx, out_w : Q8*, q_dev : Int8*, scales_dev : Float32*, k : Int32, n : Int32) : Int32
    fun q8_destroy = shainet_attn_q8_destroy(w : Q8) : Int32
    fun q8_export = shainet_attn_q8_export(w : Q8, q_host : Int8*, scales_host : Float32*) : Int32
    fun q8_gemv_dev = shainet_attn_q8_gemv_dev(ctx : Ctx, w : Q8, x_dev : Float32*, y_dev : Float32*, m : Int32,
                                               stream : Void*) : Int32
    fun block_create = shainet_attn_block_create(ctx : Ctx, out_block : Block*, kv : Kv, d_model : Int32, norm1 : Float32*,
                                                 wq : Q8, wk : Q8, wv : Q8, wo : Q8, norm2 : Float32*, gate : Q8, up : Q8,
                                                 down : Q8, eps : Float64) : Int32
    fun block_destroy = shainet_attn_block_destroy(block : Block) : Int32
    fun block_forward_dev = shainet_attn_block_forward_dev(ctx : Ctx, block : Block, x_dev : Float32*, out_dev : Float32*,
                                                           new_tokens : Int32, stream : Void*) : Int32
    fun block_forward_host = shainet_attn_block_forward_host(ctx : Ctx, block : Block, x : Float32*, out_ptr : Float32*,
                                                             new_tokens : Int32) : Int32
    fun decoder_create = shainet_attn_decoder_create(ctx : Ctx, out_dec : Decoder*, blocks : Block*, n_layers : Int32,
                                                     embedding : Float32*, vocab : Int32, final_norm : Float32*, lm_head : Q8,
                                                     lm_bias : Float32*, eps : Float64) : Int32
    fun decoder_destroy = shainet_attn_decoder_destroy(dec : Decoder) : Int32
    fun decoder_run = shainet_attn_decoder_run(ctx : Ctx, dec : Decoder, token_ids : Int32*, n_tokens : Int32,
                                               logits : Float32*, next_token : Int32*) : Int32
    fun decoder_generate = shainet_attn_decoder_generate(ctx : Ctx, dec : Decoder, prompt_ids : Int32*, n_prompt : Int32,
                                                         steps : Int32, tokens : Int32*) : Int32

    # one decode token with the split partials in a fixed array inside the library (no allocation)
    fun decode_noalloc = shainet_attn_decode_noalloc(q : Float32*, k_cache : Float32*, v_cache : Float32*, out_ptr : Float32*,
                                                     start_pos : Int32, num_heads : Int32, heads_per_kv : Int32,
                                                     head_dim : Int32, capacity : Int32, scale : Float32,
                                                     stream : Void*) : Int32
  end

  # Thin, exception-raising wrapper in the style of SHAInet::CUDA (src/shainet/cuda.cr).
  module AttnB200
    extend self

    @@ctx : LibShainetAttn::Ctx = Pointer(Void).null.as(LibShainetAttn::Ctx)

    # Replaces CUDA.fully_available? for the attention path (cuda.cr:778-780).
    def available? : Bool
      LibShainetAttn.device_count > 0
    end

    def check(rc : Int32)
      raise "libshainet_attn: #{String.new(LibShainetAttn.last_error)}" if rc < 0
      rc
    end

    # One context per process, created on first use: it stands for the class-level
    # @@gpu_staging / @@gpu_attn_out / @@gpu_attn_ws scratch (llama_block.cr:57-68).
    def ctx : LibShainetAttn::Ctx
      if @@ctx.null?
        c = Pointer(Void).null.as(LibShainetAttn::Ctx)
        check LibShainetAttn.ctx_create(pointerof(c), 0)
        @@ctx = c
      end
      @@ctx
    end
  end
end
