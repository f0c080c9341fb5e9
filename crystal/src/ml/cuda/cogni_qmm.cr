# cogni_qmm.cr -- the Crystal side of libcogni_qmm.so, the B200 (sm_100a) quantized-matmul engine.
#
# This is the file a maintainer adds next to src/ml/cuda/driver.cr.  It follows that file's style:
# a thin `lib` over a C ABI, every call returning Int32 and checked with ML::CUDA.check!
# (driver.cr:57-59), explicit `close` on every device object, no finalizers on device memory.
#
#   LibCogniQMM            one `fun` per symbol of include/cogni_qmm.h and include/cogni_qmm_diag.h
#   LibCUDADriverExt       the Driver-API calls the engine's host side needs beyond driver.cr:1-51
#                          (events, async copies, primary context, peer access, IPC handles)
#   LibNCCL                the NCCL calls of the row / vocabulary sharding
#   ML::CUDA::QuantMatmul  the call surface of ML::GGUF::QuantMatmul.matmul_add (quant_matmul.cr:20-24)
#   ML::CUDA::DeviceQuantWeight   a QuantWeight (compute.cr:20-45) resident in HBM, raw bytes verbatim
#   ML::CUDA::Qwen35DeviceWeights tensor name -> DeviceQuantWeight, mutex-guarded idempotent close
#                                 (qwen35_weights.cr:80-90, 147-160)
#   ML::CUDA::ShardedQuantWeight / ShardedLmHead   rows split over the GPUs of one box
#
# The toolchain that builds the engine has no Crystal compiler, so this file is not compiled
# there; a test parses its `fun` declarations against the C headers (names, arity, return type).

@[Link(ldflags: "-L#{__DIR__}/../../../vendor/cogni_qmm -lcogni_qmm")]
lib LibCogniQMM
  alias DevPtr = UInt64 # same value as LibCUDADriver::CUdeviceptr

  TYPE_Q8_0   =  8
  TYPE_Q4_K   = 12
  TYPE_Q5_K   = 13
  TYPE_Q6_K   = 14
  TYPE_IQ4_NL = 20
  OUT_F32     =  0
  OUT_BF16    =  1
  ERR_LIMIT        = 1006
  ERR_TIMEOUT      = 1007
  ERR_NCCL_MISSING = 1008

  struct Exchange
    world : Int32
    rank : Int32
    peer_offset : StaticArray(Int64, 8)
    epoch : UInt32*
    ticket : UInt32*
  end

  fun cogni_qmm_abi_version : Int32
  fun cogni_qmm_status_string(status : Int32) : UInt8*
  fun cogni_qmm_wait_timeouts : UInt32
  fun cogni_qmm_reset_wait_timeouts : Int32
  fun cogni_qmm_block_bytes(type : Int32) : Int32
  fun cogni_qmm_block_elements(type : Int32) : Int32
  fun cogni_qmm_row_bytes(type : Int32, in_dim : Int32) : Int64
  fun cogni_qmm_tensor_bytes(type : Int32, out_dim : Int32, in_dim : Int32) : Int64
  fun cogni_qmm_dequantize(type : Int32, w : DevPtr, n : Int64, out : DevPtr, stream : Void*) : Int32
  fun cogni_qmm_gemv(type : Int32, w : DevPtr, x : DevPtr, addend : DevPtr, addend_stride : Int64,
                     y : DevPtr, in_dim : Int32, out_dim : Int32, batch : Int32, stream : Void*) : Int32
  fun cogni_qmm_gemv_resident(type : Int32, w : DevPtr, x : DevPtr, addend : DevPtr, addend_stride : Int64,
                              y : DevPtr, in_dim : Int32, out_dim : Int32, batch : Int32, stream : Void*) : Int32
  fun cogni_qmm_gemv_many_rmsnorm(type : Int32, n_weights : Int32, w : DevPtr*, x : DevPtr,
                                  norm_weight : DevPtr, eps : Float32, addend : DevPtr*,
                                  addend_stride : Int64, y : DevPtr*, out_dims : Int32*,
                                  x_scratch : DevPtr, in_dim : Int32, batch : Int32,
                                  resident : Int32, stream : Void*) : Int32
  fun cogni_qmm_embedding_lookup(type : Int32, table : DevPtr, vocab : Int32, n_embd : Int32,
                                 token_ids : DevPtr, n_tokens : Int32, out : DevPtr, status : DevPtr,
                                 stream : Void*) : Int32
  fun cogni_qmm_gemv_top1_rmsnorm(type : Int32, w : DevPtr, x : DevPtr, norm_weight : DevPtr, eps : Float32,
                                  in_dim : Int32, out_dim : Int32, batch : Int32, index_base : Int32,
                                  scratch : DevPtr, scratch_bytes : LibC::SizeT, x_scratch : DevPtr,
                                  top_index : DevPtr, top_value : DevPtr, top_key : DevPtr,
                                  resident : Int32, stream : Void*) : Int32
  fun cogni_qmm_gemv_top2_scratch_bytes(out_dim : Int32, batch : Int32) : LibC::SizeT
  fun cogni_qmm_gemv_top2(type : Int32, w : DevPtr, x : DevPtr, in_dim : Int32, out_dim : Int32,
                          batch : Int32, index_base : Int32, scratch : DevPtr, scratch_bytes : LibC::SizeT,
                          top_index : DevPtr, top_value : DevPtr, top_key : DevPtr, resident : Int32,
                          stream : Void*) : Int32
  fun cogni_qmm_gemv_swiglu(type : Int32, w : DevPtr, gate : DevPtr, up : DevPtr, addend : DevPtr,
                            addend_stride : Int64, y : DevPtr, x_scratch : DevPtr, in_dim : Int32,
                            out_dim : Int32, batch : Int32, resident : Int32, stream : Void*) : Int32
  fun cogni_qmm_gemv_many(type : Int32, n_weights : Int32, w : DevPtr*, x : DevPtr, addend : DevPtr*,
                          addend_stride : Int64, y : DevPtr*, out_dims : Int32*, in_dim : Int32,
                          batch : Int32, resident : Int32, stream : Void*) : Int32
  fun cogni_qmm_gemv_many_exchange(type : Int32, n_weights : Int32, w : DevPtr*, x : DevPtr,
                                   addend : DevPtr*, addend_stride : Int64, y : DevPtr*, y_pitch : Int64,
                                   out_dims : Int32*, in_dim : Int32, batch : Int32, resident : Int32,
                                   exchange : Exchange*, wait_previous : Int32, stream : Void*) : Int32
  fun cogni_qmm_exchange_unpack(words : DevPtr, n : Int64, epoch : UInt32, out : DevPtr, stream : Void*) : Int32
  fun cogni_qmm_sharded_gemv_nccl(nccl_comm : Void*, world : Int32, rank : Int32, type : Int32,
                                  w_shard : DevPtr, x : DevPtr, gather : DevPtr, in_dim : Int32,
                                  rows : Int32, batch : Int32, resident : Int32, stream : Void*) : Int32
  fun cogni_qmm_sharded_top1_nccl(nccl_comm : Void*, world : Int32, type : Int32, w_shard : DevPtr,
                                  x : DevPtr, in_dim : Int32, rows : Int32, batch : Int32,
                                  index_base : Int32, scratch : DevPtr, scratch_bytes : LibC::SizeT,
                                  keys : DevPtr, top_index : DevPtr, top_value : DevPtr, stream : Void*) : Int32
  fun cogni_qmm_enable_peer_access(peer_device : Int32) : Int32
  fun cogni_qmm_gemv_top1_scratch_bytes(out_dim : Int32, batch : Int32) : LibC::SizeT
  fun cogni_qmm_gemv_top1(type : Int32, w : DevPtr, x : DevPtr, in_dim : Int32, out_dim : Int32,
                          batch : Int32, index_base : Int32, scratch : DevPtr, scratch_bytes : LibC::SizeT,
                          top_index : DevPtr, top_value : DevPtr, top_key : DevPtr, stream : Void*) : Int32
  fun cogni_qmm_gemv_top1_noalloc_max_scratch : LibC::SizeT
  fun cogni_qmm_gemv_top1_noalloc(type : Int32, w : DevPtr, x : DevPtr, in_dim : Int32, out_dim : Int32,
                                  batch : Int32, index_base : Int32, top_index : DevPtr,
                                  top_value : DevPtr, top_key : DevPtr, stream : Void*) : Int32
  fun cogni_qmm_top1_unpack_keys(keys : DevPtr, batch : Int32, top_index : DevPtr,
                                 top_value : DevPtr, stream : Void*) : Int32
  fun cogni_qmm_gemm_bf16(type : Int32, w : DevPtr, x_bf16 : DevPtr, y : DevPtr, out_type : Int32,
                          m_rows : Int32, n_out : Int32, k_in : Int32, stream : Void*) : Int32
  fun cogni_qmm_matmul_add_host(x : Float32*, rows : Int32, in_dim : Int32, w_raw : Void*,
                                w_bytes : Int64, type : Int32, out_dim : Int32, bias : Float32*,
                                y : Float32*) : Int32
  # include/cogni_qmm_diag.h
  fun cogni_qmm_set_kernel_choice(choice : Int32) : Int32
  fun cogni_qmm_diag_expire_wait(limit_us : UInt32, stream : Void*) : Int32
end

# Driver-API calls beyond the 28 of driver.cr:1-51 that the engine's host side uses.
@[Link(ldflags: "-lcuda")]
lib LibCUDADriverExt
  alias CUevent = Void*

  struct CUipcMemHandle
    reserved : StaticArray(UInt8, 64)
  end

  fun cuDevicePrimaryCtxRetain(ctx : Void**, dev : Int32) : Int32
  fun cuDevicePrimaryCtxRelease_v2(dev : Int32) : Int32
  fun cuCtxSetCurrent(ctx : Void*) : Int32
  fun cuDeviceGetAttribute(pi : Int32*, attrib : Int32, dev : Int32) : Int32
  fun cuEventCreate(event : CUevent*, flags : UInt32) : Int32
  fun cuEventRecord(event : CUevent, stream : Void*) : Int32
  fun cuEventSynchronize(event : CUevent) : Int32
  fun cuEventElapsedTime(ms : Float32*, start : CUevent, stop : CUevent) : Int32
  fun cuEventDestroy_v2(event : CUevent) : Int32
  fun cuMemcpyHtoDAsync_v2(dst : UInt64, src : Void*, bytesize : LibC::SizeT, stream : Void*) : Int32
  fun cuMemcpyDtoHAsync_v2(dst : Void*, src : UInt64, bytesize : LibC::SizeT, stream : Void*) : Int32
  fun cuMemsetD8_v2(dst : UInt64, value : UInt8, n : LibC::SizeT) : Int32
  fun cuMemHostAlloc(pp : Void**, bytesize : LibC::SizeT, flags : UInt32) : Int32
  fun cuMemFreeHost(p : Void*) : Int32
  fun cuDeviceCanAccessPeer(can : Int32*, dev : Int32, peer : Int32) : Int32
  fun cuCtxEnablePeerAccess(peer_ctx : Void*, flags : UInt32) : Int32
  fun cuIpcGetMemHandle(handle : CUipcMemHandle*, dptr : UInt64) : Int32
  fun cuIpcOpenMemHandle_v2(pdptr : UInt64*, handle : CUipcMemHandle, flags : UInt32) : Int32
  fun cuIpcCloseMemHandle(dptr : UInt64) : Int32
end

@[Link(ldflags: "-lnccl")]
lib LibNCCL
  alias Comm = Void*

  struct UniqueId
    internal : StaticArray(UInt8, 128)
  end

  fun ncclGetUniqueId(id : UniqueId*) : Int32
  fun ncclCommInitRank(comm : Comm*, nranks : Int32, id : UniqueId, rank : Int32) : Int32
  fun ncclCommInitAll(comms : Comm*, ndev : Int32, devlist : Int32*) : Int32
  fun ncclCommDestroy(comm : Comm) : Int32
  fun ncclCommAbort(comm : Comm) : Int32
  fun ncclGetErrorString(result : Int32) : UInt8*
end

# Suffix => QuantWeight views of the reference's per-layer weight structs (qwen35_weights.cr:162-199),
# so that a device map can be keyed by GGUF tensor name.
module ML::GGUF
  struct Qwen35RecurrentWeights
    def quant_weights : Hash(String, QuantWeight)
      {"attn_qkv" => attn_qkv_qw, "attn_gate" => attn_gate_qw, "ssm_alpha" => ssm_alpha_qw,
       "ssm_beta" => ssm_beta_qw, "ssm_out" => ssm_out_qw, "ffn_gate" => ffn_gate_qw,
       "ffn_up" => ffn_up_qw, "ffn_down" => ffn_down_qw}
    end
  end

  struct Qwen35FullAttnWeights
    def quant_weights : Hash(String, QuantWeight)
      {"attn_q" => attn_q_qw, "attn_k" => attn_k_qw, "attn_v" => attn_v_qw,
       "attn_output" => attn_output_qw, "ffn_gate" => ffn_gate_qw, "ffn_up" => ffn_up_qw,
       "ffn_down" => ffn_down_qw}
    end
  end
end

module ML::CUDA
  # check! for the engine's statuses: the reference's message plus the engine's own text.
  def self.qmm_check!(code : Int32, what : String) : Nil
    return if code == 0
    raise "#{what} failed with status #{code} (#{String.new(LibCogniQMM.cogni_qmm_status_string(code))})"
  end

  module QuantMatmul
    # Same signature as ML::GGUF::QuantMatmul.matmul_add (src/ml/gguf/quant_matmul.cr:20-24):
    # one-shot upload, device GEMV, read back; bias is the accumulator start.
    def self.matmul_add(x : Array(Float32), rows : Int32, in_dim : Int32, w_raw : Bytes,
                        w_type : ML::GGUF::TensorType, out_dim : Int32, bias : Array(Float32)) : Array(Float32)
      raise ArgumentError.new("x.size must be rows * in_dim") unless x.size == rows * in_dim
      raise ArgumentError.new("bias.size must be out_dim") unless bias.size == out_dim
      y = Array(Float32).new(rows * out_dim, 0.0_f32)
      ML::CUDA.qmm_check! LibCogniQMM.cogni_qmm_matmul_add_host(x.to_unsafe, rows, in_dim,
        w_raw.to_unsafe.as(Void*), w_raw.size.to_i64, w_type.value.to_i32, out_dim,
        bias.to_unsafe, y.to_unsafe), "cogni_qmm_matmul_add_host"
      y
    end
  end

  # A quantized weight resident in HBM: the verbatim GGUF bytes of rows [row_begin, row_end), as
  # QwenRecurrentLayerRunner#upload_weights leaves them (qwen_recurrent_layer_runner.cr:570-587).
  class DeviceQuantWeight
    getter buffer : DeviceBuffer
    getter type : ML::GGUF::TensorType
    getter out_dim : Int32
    getter in_dim : Int32
    getter row_begin : Int32
    @top1_scratch : DeviceBuffer?

    def self.upload(qw : ML::GGUF::QuantWeight, row_begin : Int32 = 0, row_end : Int32? = nil) : self
      last = row_end || qw.out_dim
      rb = LibCogniQMM.cogni_qmm_row_bytes(qw.type.value.to_i32, qw.in_dim)
      raise ArgumentError.new("in_dim is not a multiple of the block size") if rb < 0
      slice = qw.raw[row_begin.to_i64 * rb, (last - row_begin).to_i64 * rb]
      buf = DeviceBuffer.new(LibC::SizeT.new(slice.size))
      ML::CUDA.copy_htod!(buf, slice, "upload #{qw.route_tag}")
      new(buf, qw.type, last - row_begin, qw.in_dim, row_begin)
    end

    def initialize(@buffer, @type, @out_dim, @in_dim, @row_begin)
      @closed = false
    end

    # y[b, :] = addend + W x[b, :]; addend_stride 0 = bias, out_dim = residual (the *_gemv_add_* kernels).
    def gemv(x : DeviceBuffer, y : DeviceBuffer, batch : Int32, addend : DeviceBuffer? = nil,
             addend_stride : Int64 = 0_i64, stream : Void* = ML::CUDA.current_stream) : Nil
      ML::CUDA.qmm_check! LibCogniQMM.cogni_qmm_gemv_resident(@type.value.to_i32, @buffer.ptr, x.ptr,
        addend ? addend.ptr : 0_u64, addend_stride, y.ptr, @in_dim, @out_dim, batch, stream), "cogni_qmm_gemv"
    end

    # Fused lm_head: argmax per batch row without writing logits; indices are global (row_begin added).
    def gemv_top1(x : DeviceBuffer, batch : Int32, top_index : DeviceBuffer, top_value : DeviceBuffer,
                  top_key : DeviceBuffer? = nil, stream : Void* = ML::CUDA.current_stream) : Nil
      need = LibCogniQMM.cogni_qmm_gemv_top1_scratch_bytes(@out_dim, batch)
      scratch = @top1_scratch
      if scratch.nil? || scratch.bytesize < need
        scratch.try &.close
        scratch = DeviceBuffer.new(need)
        ML::CUDA.check! LibCUDADriverExt.cuMemsetD8_v2(scratch.ptr, 0_u8, need), "cuMemsetD8(top1 scratch)"
        @top1_scratch = scratch
      end
      ML::CUDA.qmm_check! LibCogniQMM.cogni_qmm_gemv_top1(@type.value.to_i32, @buffer.ptr, x.ptr, @in_dim,
        @out_dim, batch, @row_begin, scratch.ptr, scratch.bytesize, top_index.ptr, top_value.ptr,
        top_key ? top_key.ptr : 0_u64, stream), "cogni_qmm_gemv_top1"
    end

    # Prefill: y[m, n] = sum_k x[m, k] * bf16(dequant(W[n, k])), x bf16 [m_rows, in_dim].
    def gemm(x_bf16 : DeviceBuffer, y : DeviceBuffer, m_rows : Int32, out_bf16 : Bool = false,
             stream : Void* = ML::CUDA.current_stream) : Nil
      ML::CUDA.qmm_check! LibCogniQMM.cogni_qmm_gemm_bf16(@type.value.to_i32, @buffer.ptr, x_bf16.ptr, y.ptr,
        out_bf16 ? LibCogniQMM::OUT_BF16 : LibCogniQMM::OUT_F32, m_rows, @out_dim, @in_dim, stream),
        "cogni_qmm_gemm_bf16"
    end

    def close : Nil
      return if @closed
      @top1_scratch.try &.close
      @buffer.close
      @closed = true
    end
  end

  # Tensor name -> DeviceQuantWeight for a loaded Qwen35Weights; keeps the weight set (and with it
  # the mmap) alive until close, which is idempotent and safe to call from several fibers.
  class Qwen35DeviceWeights
    @weights = {} of String => DeviceQuantWeight
    @close_mutex = Mutex.new
    @closed = false

    def initialize(@host : ML::GGUF::Qwen35Weights, rank : Int32 = 0, world : Int32 = 1)
      add = ->(name : String, qw : ML::GGUF::QuantWeight) do
        rows = qw.out_dim // world
        r0 = world > 1 ? rank * rows : 0
        r1 = world > 1 ? r0 + rows : qw.out_dim
        @weights[name] = DeviceQuantWeight.upload(qw, r0, r1)
      end
      add.call("token_embd.weight", @host.token_embd)
      add.call("output.weight", @host.output)
      @host.layers.each_with_index do |layer, il|
        layer.quant_weights.each { |suffix, qw| add.call("blk.#{il}.#{suffix}.weight", qw) }
      end
    end

    def [](name : String) : DeviceQuantWeight
      @weights[name]? || raise "qwen35_weights: missing tensor #{name.inspect}"
    end

    def close : Nil
      @close_mutex.synchronize do
        return if @closed
        @weights.each_value &.close
        @weights.clear
        @host.close
        @closed = true
      end
    end
  end

  # Rows [rank * N / world, (rank + 1) * N / world) of a weight on this GPU; the exchange step is an
  # in-place ncclAllGather into a [world][batch][rows] buffer.
  class ShardedQuantWeight
    getter local : DeviceQuantWeight
    getter world : Int32
    getter rank : Int32

    def initialize(qw : ML::GGUF::QuantWeight, @comm : LibNCCL::Comm, @world : Int32, @rank : Int32)
      raise ArgumentError.new("out_dim must divide evenly over the ranks") unless qw.out_dim % @world == 0
      rows = qw.out_dim // @world
      @local = DeviceQuantWeight.upload(qw, @rank * rows, (@rank + 1) * rows)
    end

    def gemv(x : DeviceBuffer, gather : DeviceBuffer, batch : Int32, stream : Void* = ML::CUDA.current_stream) : Nil
      ML::CUDA.qmm_check! LibCogniQMM.cogni_qmm_sharded_gemv_nccl(@comm, @world, @rank,
        @local.type.value.to_i32, @local.buffer.ptr, x.ptr, gather.ptr, @local.in_dim, @local.out_dim,
        batch, 1, stream), "cogni_qmm_sharded_gemv_nccl"
    end

    def close : Nil
      @local.close
    end
  end

  # Vocabulary-sharded lm_head: per-shard fused top-1, one ncclAllReduce(ncclMax) on the int64 keys
  # (highest value, lowest index: qwen35_cpu.cr:2052-2055).
  class ShardedLmHead
    getter local : DeviceQuantWeight

    def initialize(qw : ML::GGUF::QuantWeight, @comm : LibNCCL::Comm, @world : Int32, @rank : Int32)
      rows = qw.out_dim // @world
      last = @rank == @world - 1 ? qw.out_dim : (@rank + 1) * rows
      @local = DeviceQuantWeight.upload(qw, @rank * rows, last)
      @scratch = DeviceBuffer.new(LibCogniQMM.cogni_qmm_gemv_top1_scratch_bytes(@local.out_dim, 16))
      ML::CUDA.check! LibCUDADriverExt.cuMemsetD8_v2(@scratch.ptr, 0_u8, @scratch.bytesize), "cuMemsetD8"
    end

    def top1(x : DeviceBuffer, batch : Int32, keys : DeviceBuffer, top_index : DeviceBuffer,
             top_value : DeviceBuffer, stream : Void* = ML::CUDA.current_stream) : Nil
      ML::CUDA.qmm_check! LibCogniQMM.cogni_qmm_sharded_top1_nccl(@comm, @world, @local.type.value.to_i32,
        @local.buffer.ptr, x.ptr, @local.in_dim, @local.out_dim, batch, @local.row_begin, @scratch.ptr,
        @scratch.bytesize, keys.ptr, top_index.ptr, top_value.ptr, stream), "cogni_qmm_sharded_top1_nccl"
    end

    def close : Nil
      @scratch.close
      @local.close
    end
  end
end
