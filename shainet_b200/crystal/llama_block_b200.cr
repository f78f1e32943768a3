# Patch of SHAInet::LlamaBlock (src/shainet/transformer/llama_block.cr) that routes
# the cached attention through libshainet_attn.  Public API is unchanged:
# LlamaBlock.new(...), #forward, #forward_cached, #clear_cache!, #to_gpu!,
# #finalize and every property keep their signatures.  Only the private
# attention_cached_cpu / gpu_attention? / clear_cache! / finalize bodies change;
# attention_heads_gpu, ensure_gpu_cache!, grow_dev_buf and the @@gpu_* class
# variables (llama_block.cr:57-68, 407-479, 497-530) are no longer needed.
#
# Not compiled here (no Crystal compiler on the build image); it is the change a
# maintainer would make, written against the reference's own code.
require "./shainet_attn"

module SHAInet
  class LlamaBlock < MatrixLayer
    @attn_kv : LibShainetAttn::Kv = Pointer(Void).null.as(LibShainetAttn::Kv)
    @attn_params_dirty : Bool = true

    # Call after changing rope_theta / rope_freqs / q_norm / k_norm / b_q / b_k / b_v
    # (the loader sets them after construction, hf_loader.cr:321-373).
    def attn_params_changed!
      @attn_params_dirty = true
    end

    private def attn_kv : LibShainetAttn::Kv
      if @attn_kv.null?
        kv = Pointer(Void).null.as(LibShainetAttn::Kv)
        AttnB200.check LibShainetAttn.kv_create(AttnB200.ctx, pointerof(kv), @num_heads, @num_kv_heads, @head_dim, 256)
        @attn_kv = kv
        @attn_params_dirty = true
      end
      if @attn_params_dirty
        # inv_freq stays computed by Crystal (llama_block.cr:669-675), so rope_theta,
        # rope_freqs and LLaMA-3 scaling keep their exact semantics.
        half = @head_dim // 2
        freqs = Array(Float32).new(half) { |i| inv_freq(i) }
        AttnB200.check LibShainetAttn.kv_set_rope(@attn_kv, freqs.to_unsafe, half)
        qn = @q_norm.try(&.to_unsafe) || Pointer(Float32).null
        kn = @k_norm.try(&.to_unsafe) || Pointer(Float32).null
        AttnB200.check LibShainetAttn.kv_set_qk_norm(@attn_kv, qn, kn, @qk_norm_eps)
        bq = @b_q.try(&.to_unsafe) || Pointer(Float32).null
        bk = @b_k.try(&.to_unsafe) || Pointer(Float32).null
        bv = @b_v.try(&.to_unsafe) || Pointer(Float32).null
        AttnB200.check LibShainetAttn.kv_set_bias(@attn_kv, bq, bk, bv)
        @attn_params_dirty = false
      end
      @attn_kv
    end

    def clear_cache!
      @k_cache.each(&.clear)
      @v_cache.each(&.clear)
      @cache_len = 0
      LibShainetAttn.kv_reset(@attn_kv) unless @attn_kv.null?
    end

    def finalize
      LibShainetAttn.kv_destroy(@attn_kv) unless @attn_kv.null?
    end

    private def gpu_attention? : Bool
      return false if force_cpu_attention?
      avail = @gpu_attn_avail
      if avail.nil?
        avail = !ENV["SHAINET_CPU_ATTENTION"]? && AttnB200.available?
        @gpu_attn_avail = avail
      end
      avail
    end

    # Replaces llama_block.cr:246-299.  The projections stay where they are; bias,
    # QK-norm, RoPE, the cache append and the attention all happen in one library
    # call on the raw projection outputs.
    private def attention_cached_cpu(x : SimpleMatrix) : SimpleMatrix
      # Without a device (or with force_cpu_attention / SHAINET_CPU_ATTENTION=1) the
      # reference's own definition runs: bias, QK-norm, host K-RoPE + append,
      # attention_heads_cpu.
      return previous_def unless gpu_attention?
      new_tokens = x.rows
      scale = (1.0 / Math.sqrt(@head_dim.to_f64)).to_f32
      q_full = gpu_matmul(x, @w_q)
      k_new = gpu_matmul(x, @w_k)
      v_new = gpu_matmul(x, @w_v)
      output = SimpleMatrix.new(new_tokens, @q_dim)
      AttnB200.check LibShainetAttn.forward_host(AttnB200.ctx, attn_kv, q_full.data.to_unsafe, k_new.data.to_unsafe,
        v_new.data.to_unsafe, output.data.to_unsafe, new_tokens, scale, 0_u32)
      @cache_len += new_tokens
      gpu_matmul(output, @w_o)
    end

    # ---- second level: the whole forward_cached on the device (llama_block.cr:189-196) ----
    # Available once every projection and the FFN are Q8_0 on the device (to_gpu!(quantize: true),
    # llama_block.cr:132-176) and the FFN is the dense SwiGLU; otherwise the definition above runs.
    @attn_block : LibShainetAttn::Block = Pointer(Void).null.as(LibShainetAttn::Block)

    private def q8_handle(w) : LibShainetAttn::Q8
      qm = w.as(QuantizedCudaMatrix)
      h = Pointer(Void).null.as(LibShainetAttn::Q8)
      # adopts the arrays the QuantizedCudaMatrix owns: q [cols, rows] int8, scales [cols, blocks]
      AttnB200.check LibShainetAttn.q8_wrap(AttnB200.ctx, pointerof(h), qm.q_ptr, qm.scale_ptr, qm.rows, qm.cols)
      h
    end

    private def attn_block? : Bool
      return false unless gpu_attention?
      return true unless @attn_block.null?
      ws = {@w_q, @w_k, @w_v, @w_o}
      return false unless ws.all?(QuantizedCudaMatrix)
      f = @ffn
      return false unless f.is_a?(SwiGLUFF) && {f.gate_proj, f.up_proj, f.down_proj}.all?(QuantizedCudaMatrix)
      blk = Pointer(Void).null.as(LibShainetAttn::Block)
      AttnB200.check LibShainetAttn.block_create(AttnB200.ctx, pointerof(blk), attn_kv, @d_model,
        @norm1.gamma.as(SimpleMatrix).data.to_unsafe, q8_handle(@w_q), q8_handle(@w_k), q8_handle(@w_v), q8_handle(@w_o),
        @norm2.gamma.as(SimpleMatrix).data.to_unsafe, q8_handle(f.gate_proj), q8_handle(f.up_proj), q8_handle(f.down_proj),
        @qk_norm_eps)   # LlamaBlock.new hands the same eps to norm1, norm2 and the per-head norms (llama_block.cr:92-94)
      @attn_block = blk
      true
    end

    def forward_cached(x : SimpleMatrix) : SimpleMatrix
      return previous_def unless attn_block?
      out = SimpleMatrix.new(x.rows, x.cols)
      AttnB200.check LibShainetAttn.block_forward_host(AttnB200.ctx, @attn_block, x.data.to_unsafe, out.data.to_unsafe, x.rows)
      @cache_len += x.rows
      out
    end
  end
end
