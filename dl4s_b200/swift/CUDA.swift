//  CUDA.swift — a CUDA DeviceType for DL4S on top of libdl4s_cuda.so.
//
//  Goes to Sources/DL4S/Engine/CUDA/CUDA.swift of a DL4S checkout, next to
//  Engine/CPU and Engine/GPU. It has NOT been compiled: no Swift toolchain was
//  available where this library was built. It is the mechanical glue between
//  DL4S's protocols (Engine/Engine.swift:30-581) and the C ABI in dl4s_cuda.h;
//  the ABI itself is exercised by the Python mirror in dl4s_b200/cuda.py,
//  which makes the same calls in the same order.
//
//  Build: add `.target(name: "CDL4SCUDA")` to Package.swift, list it in the
//  DL4S target's dependencies and pass `-Xlinker -L<dir of libdl4s_cuda.so>`.

#if canImport(CDL4SCUDA)
import Foundation
import CDL4SCUDA

@inline(__always)
private func check(_ status: dl4s_status, _ what: StaticString = #function) {
    // DL4S aborts on violated preconditions (e.g. Matrix.swift:39-41); keep that behaviour.
    if status != DL4S_OK {
        fatalError("\(what): \(String(cString: dl4s_cuda_last_error()))")
    }
}

public struct CUDA: DeviceType {
    public typealias Memory = CUDAMemoryOperators
    public typealias Engine = CUDAEngine

    /// Arithmetic of the fused hooks: DL4S_PREC_F16 (tensor cores) or DL4S_PREC_FP32.
    public static var precision: Int32 = Int32(DL4S_PREC_F16)

    static let ready: Bool = {
        check(dl4s_cuda_init(nil, 0))
        return true
    }()
}

/// Device address + size; Hashable as MemoryOperatorsType.RawBuffer requires (Engine.swift:41).
public struct CUDABuffer: Hashable {
    var address: UInt
    var byteCount: Int
    var pointer: UnsafeMutableRawPointer? { UnsafeMutableRawPointer(bitPattern: address) }
    func floats() -> UnsafeMutablePointer<Float>? { pointer?.assumingMemoryBound(to: Float.self) }
}

public struct CUDAMemoryOperators: MemoryOperatorsType {
    public typealias RawBuffer = CUDABuffer
    public typealias Device = CUDA

    public static func allocateBuffer<Element>(withCapacity capacity: Int, type: Element.Type) -> Buffer<Element, CUDA> {
        _ = CUDA.ready
        var p: UnsafeMutableRawPointer? = nil
        let bytes = capacity * MemoryLayout<Element>.stride
        check(dl4s_cuda_malloc(bytes, &p))
        return Buffer(memory: CUDABuffer(address: UInt(bitPattern: p), byteCount: bytes))
    }

    public static func allocateBuffer<Element>(withShape shape: [Int], type: Element.Type) -> ShapedBuffer<Element, CUDA> {
        ShapedBuffer(values: allocateBuffer(withCapacity: shape.reduce(1, *), type: Element.self), shape: shape)
    }

    // Only root buffers reach free (TensorHandle.deinit, Tensor.swift:38-42); the free is stream-ordered.
    public static func free<Element>(_ buffer: Buffer<Element, CUDA>) { check(dl4s_cuda_free(buffer.memory.pointer)) }
    public static func free<Element>(_ buffer: ShapedBuffer<Element, CUDA>) { free(buffer.values) }

    public static func assign<Element>(from source: UnsafeBufferPointer<Element>, to destination: Buffer<Element, CUDA>, count: Int) {
        check(dl4s_cuda_memcpy_h2d(destination.memory.pointer, source.baseAddress, count * MemoryLayout<Element>.stride))
    }
    public static func assign<Element>(from source: Buffer<Element, CUDA>, to destination: Buffer<Element, CUDA>, count: Int) {
        check(dl4s_cuda_memcpy_d2d(destination.memory.pointer, source.memory.pointer, count * MemoryLayout<Element>.stride))
    }
    public static func assign<Element>(from source: Buffer<Element, CUDA>, to destination: UnsafeMutableBufferPointer<Element>, count: Int) {
        check(dl4s_cuda_memcpy_d2h(destination.baseAddress, source.memory.pointer, count * MemoryLayout<Element>.stride))
    }

    public static func getValue<Element>(from source: Buffer<Element, CUDA>) -> Element {
        let tmp = UnsafeMutablePointer<Element>.allocate(capacity: 1)
        defer { tmp.deallocate() }
        check(dl4s_cuda_memcpy_d2h(tmp, source.memory.pointer, MemoryLayout<Element>.stride))
        return tmp.pointee
    }
    public static func setPointee<Element>(of buffer: Buffer<Element, CUDA>, to newValue: Element) {
        var v = newValue
        check(dl4s_cuda_memcpy_h2d(buffer.memory.pointer, &v, MemoryLayout<Element>.stride))
    }
    public static func getSize<Element>(of buffer: Buffer<Element, CUDA>) -> Int {
        buffer.memory.byteCount / MemoryLayout<Element>.stride
    }
    public static func advance<Element>(buffer: Buffer<Element, CUDA>, by advancement: Int) -> Buffer<Element, CUDA> {
        let off = advancement * MemoryLayout<Element>.stride
        return Buffer(memory: CUDABuffer(address: buffer.memory.address + UInt(off), byteCount: buffer.memory.byteCount - off))
    }

    // get / set(slice:) — a leading-prefix index is a view, anything else a strided copy
    // through dl4s_cuda_copy_strided_f32, exactly as CPU.swift:137-213 does with memcpy loops.
    public static func get<Element>(slice: [Int?], of buffer: Buffer<Element, CUDA>, with shape: [Int]) -> (Buffer<Element, CUDA>, Bool, [Int]) {
        let strides = MemoryOps.strides(from: shape)
        let idx = slice + [Int?](repeating: nil, count: shape.count - slice.count)
        let lead = idx.prefix(while: { $0 != nil }).count
        if idx[lead...].allSatisfy({ $0 == nil }) {
            let off = (0 ..< lead).map { idx[$0]! * strides[$0] }.reduce(0, +)
            return (advance(buffer: buffer, by: off), false, Array(shape[lead...]))
        }
        let keep = idx.indices.filter { idx[$0] == nil }
        let off = idx.indices.filter { idx[$0] != nil }.map { idx[$0]! * strides[$0] }.reduce(0, +)
        let outShape = keep.map { shape[$0] }
        let out: Buffer<Element, CUDA> = allocateBuffer(withCapacity: outShape.reduce(1, *), type: Element.self)
        let src = keep.map { Int64(strides[$0]) }, dst = MemoryOps.strides(from: outShape).map(Int64.init), ext = outShape.map(Int64.init)
        check(dl4s_cuda_copy_strided_f32(buffer.memory.floats(), src, Int64(off), out.memory.floats(), dst, 0, ext, Int32(ext.count)))
        return (out, true, outShape)
    }
    public static func get<Element>(slice: [CountableRange<Int>?], of buffer: Buffer<Element, CUDA>, with shape: [Int]) -> (Buffer<Element, CUDA>, Bool, [Int]) {
        let strides = MemoryOps.strides(from: shape)
        let rng = slice + [CountableRange<Int>?](repeating: nil, count: shape.count - slice.count)
        let lo = rng.indices.map { rng[$0]?.lowerBound ?? 0 }, ext = rng.indices.map { rng[$0]?.count ?? shape[$0] }
        let off = zip(lo, strides).map(*).reduce(0, +)
        let out: Buffer<Element, CUDA> = allocateBuffer(withCapacity: ext.reduce(1, *), type: Element.self)
        check(dl4s_cuda_copy_strided_f32(buffer.memory.floats(), strides.map(Int64.init), Int64(off), out.memory.floats(),
                                         MemoryOps.strides(from: ext).map(Int64.init), 0, ext.map(Int64.init), Int32(ext.count)))
        return (out, true, ext)
    }
    public static func set<Element>(slice: [Int?], of buffer: Buffer<Element, CUDA>, with dstShape: [Int], from source: Buffer<Element, CUDA>, with sourceShape: [Int]) {
        let strides = MemoryOps.strides(from: dstShape)
        let idx = slice + [Int?](repeating: nil, count: dstShape.count - slice.count)
        let keep = idx.indices.filter { idx[$0] == nil }
        let off = idx.indices.filter { idx[$0] != nil }.map { idx[$0]! * strides[$0] }.reduce(0, +)
        let ext = keep.map { dstShape[$0] }
        check(dl4s_cuda_copy_strided_f32(source.memory.floats(), MemoryOps.strides(from: ext).map(Int64.init), 0, buffer.memory.floats(),
                                         keep.map { Int64(strides[$0]) }, Int64(off), ext.map(Int64.init), Int32(ext.count)))
    }
    public static func set<Element>(slice: [Range<Int>?], of buffer: Buffer<Element, CUDA>, with dstShape: [Int], from source: Buffer<Element, CUDA>, with sourceShape: [Int]) {
        let strides = MemoryOps.strides(from: dstShape)
        let rng = slice + [Range<Int>?](repeating: nil, count: dstShape.count - slice.count)
        let lo = rng.indices.map { rng[$0]?.lowerBound ?? 0 }, ext = rng.indices.map { rng[$0]?.count ?? dstShape[$0] }
        check(dl4s_cuda_copy_strided_f32(source.memory.floats(), MemoryOps.strides(from: ext).map(Int64.init), 0, buffer.memory.floats(),
                                         strides.map(Int64.init), Int64(zip(lo, strides).map(*).reduce(0, +)), ext.map(Int64.init), Int32(ext.count)))
    }
}

/// EngineType for CUDA. Only Float is accelerated (the attention path is fp32);
/// other element types and the operations outside the path abort with a clear message,
/// as DL4S's own unfinished engine entries do (CPUEngine.swift:856, GPU.swift:72).
public struct CUDAEngine: EngineType {
    public typealias Device = CUDA

    @inline(__always) private static func f<N>(_ b: Buffer<N, CUDA>) -> UnsafeMutablePointer<Float>? {
        precondition(N.self == Float.self, "the CUDA device implements Float only")
        return b.memory.floats()
    }
    @inline(__always) private static func s(_ shape: [Int]) -> [Int64] { shape.map(Int64.init) }

    public static func fill<N: NumericType>(value: N, result: Buffer<N, CUDA>, count: Int) {
        check(dl4s_cuda_fill_f32(value as! Float, f(result), Int64(count)))
    }
    public static func vAdd<N: NumericType>(lhs: Buffer<N, CUDA>, rhs: Buffer<N, CUDA>, result: Buffer<N, CUDA>, count: Int) { check(dl4s_cuda_vadd(f(lhs), f(rhs), f(result), Int64(count))) }
    public static func vSub<N: NumericType>(lhs: Buffer<N, CUDA>, rhs: Buffer<N, CUDA>, result: Buffer<N, CUDA>, count: Int) { check(dl4s_cuda_vsub(f(lhs), f(rhs), f(result), Int64(count))) }
    public static func vMul<N: NumericType>(lhs: Buffer<N, CUDA>, rhs: Buffer<N, CUDA>, result: Buffer<N, CUDA>, count: Int) { check(dl4s_cuda_vmul(f(lhs), f(rhs), f(result), Int64(count))) }
    public static func vDiv<N: NumericType>(lhs: Buffer<N, CUDA>, rhs: Buffer<N, CUDA>, result: Buffer<N, CUDA>, count: Int) { check(dl4s_cuda_vdiv(f(lhs), f(rhs), f(result), Int64(count))) }
    public static func vNeg<N: NumericType>(val: Buffer<N, CUDA>, result: Buffer<N, CUDA>, count: Int) { check(dl4s_cuda_vneg(f(val), f(result), Int64(count))) }

    public static func gemm<N: NumericType>(lhs: ShapedBuffer<N, CUDA>, rhs: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>, alpha: N, beta: N, transposeFirst: Bool, transposeSecond: Bool) {
        let M = result.shape[0], Nn = result.shape[1], K = transposeFirst ? lhs.shape[0] : lhs.shape[1]
        check(dl4s_cuda_gemm(f(lhs.values), f(rhs.values), f(result.values), Int64(M), Int64(Nn), Int64(K), alpha as! Float, beta as! Float,
                             transposeFirst ? 1 : 0, transposeSecond ? 1 : 0, CUDA.precision))
    }
    public static func band<N: NumericType>(buffer: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>, belowDiagonal: Int?, aboveDiagonal: Int?) {
        check(dl4s_cuda_band(f(buffer.values), Int64(buffer.shape[0]), Int64(buffer.shape[1]), Int32(belowDiagonal ?? 0), belowDiagonal == nil ? 0 : 1,
                             Int32(aboveDiagonal ?? 0), aboveDiagonal == nil ? 0 : 1, f(result.values)))
    }
    public static func broadcastAdd<N: NumericType>(lhs: ShapedBuffer<N, CUDA>, rhs: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>) { check(dl4s_cuda_broadcast_add(f(lhs.values), s(lhs.shape), Int32(lhs.dim), f(rhs.values), s(rhs.shape), Int32(rhs.dim), f(result.values))) }
    public static func broadcastSub<N: NumericType>(lhs: ShapedBuffer<N, CUDA>, rhs: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>) { check(dl4s_cuda_broadcast_sub(f(lhs.values), s(lhs.shape), Int32(lhs.dim), f(rhs.values), s(rhs.shape), Int32(rhs.dim), f(result.values))) }
    public static func broadcastMul<N: NumericType>(lhs: ShapedBuffer<N, CUDA>, rhs: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>) { check(dl4s_cuda_broadcast_mul(f(lhs.values), s(lhs.shape), Int32(lhs.dim), f(rhs.values), s(rhs.shape), Int32(rhs.dim), f(result.values))) }
    public static func broadcastDiv<N: NumericType>(lhs: ShapedBuffer<N, CUDA>, rhs: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>) { check(dl4s_cuda_broadcast_div(f(lhs.values), s(lhs.shape), Int32(lhs.dim), f(rhs.values), s(rhs.shape), Int32(rhs.dim), f(result.values))) }

    public static func reduceSum<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>, axes: [Int]) {
        check(dl4s_cuda_reduce_sum(f(values.values), s(values.shape), Int32(values.dim), axes.map(Int32.init), Int32(axes.count), f(result.values)))
    }
    public static func reduceSum<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>, axis: Int) { reduceSum(values: values, result: result, axes: [axis]) }
    public static func reduceMax<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>, context: ShapedBuffer<Int32, CUDA>?, axes: [Int]) {
        let ctx = context?.values.memory.pointer?.assumingMemoryBound(to: Int32.self)
        check(dl4s_cuda_reduce_max(f(values.values), s(values.shape), Int32(values.dim), axes.map(Int32.init), Int32(axes.count), f(result.values), ctx))
    }
    public static func reduceMax<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>, context: ShapedBuffer<Int32, CUDA>?, axis: Int) { reduceMax(values: values, result: result, context: context, axes: [axis]) }

    public static func exp<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>) { check(dl4s_cuda_exp(f(values.values), f(result.values), Int64(values.count))) }
    public static func log<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>) { check(dl4s_cuda_log(f(values.values), f(result.values), Int64(values.count))) }
    public static func sqrt<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>) { check(dl4s_cuda_sqrt(f(values.values), f(result.values), Int64(values.count))) }
    public static func relu<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>) { check(dl4s_cuda_relu(f(values.values), f(result.values), Int64(values.count))) }
    public static func heaviside<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>) { check(dl4s_cuda_heaviside(f(values.values), f(result.values), Int64(values.count))) }
    public static func sin<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>) { check(dl4s_cuda_sin(f(values.values), f(result.values), Int64(values.count))) }
    public static func cos<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>) { check(dl4s_cuda_cos(f(values.values), f(result.values), Int64(values.count))) }
    public static func tanh<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>) { check(dl4s_cuda_tanh(f(values.values), f(result.values), Int64(values.count))) }

    public static func permuteAxes<N: NumericType>(values: ShapedBuffer<N, CUDA>, result: ShapedBuffer<N, CUDA>, arangement: [Int]) {
        check(dl4s_cuda_permute_axes(f(values.values), s(values.shape), Int32(values.dim), arangement.map(Int32.init), f(result.values)))
    }
    public static func stack<N>(buffers: [ShapedBuffer<N, CUDA>], result: ShapedBuffer<N, CUDA>, axis: Int) {
        let ptrs: [UnsafePointer<Float>?] = buffers.map { UnsafePointer($0.values.memory.floats()) }
        let shapes = buffers.flatMap { $0.shape.map(Int64.init) }
        check(dl4s_cuda_stack(ptrs, shapes, Int32(buffers.count), Int32(buffers[0].dim), Int32(axis), result.values.memory.floats()))
    }

    public static func unstack<N>(stacked: ShapedBuffer<N, CUDA>, result: [ShapedBuffer<N, CUDA>], axis: Int) {
        let ptrs: [UnsafeMutablePointer<Float>?] = result.map { $0.values.memory.floats() }
        let shapes = result.flatMap { $0.shape.map(Int64.init) }
        check(dl4s_cuda_unstack(stacked.values.memory.floats(), ptrs, shapes, Int32(result.count), Int32(result[0].dim), Int32(axis)))
    }

    // Every remaining EngineType requirement (diagonals, min, scatter/gather, reverse,
    // img2col, subscript ops, tan/sinh/cosh, arange ...) is outside the attention path:
    //     fatalError("\(#function) is not available on the CUDA device")
    // one line each, omitted here for brevity of the glue.
}

// MARK: fused hooks
// ScaledDotProductAttention / MultiHeadAttention / LayerNorm / PointwiseFeedForward / TransformerEncoder call
// these instead of composing primitives when Device == CUDA. The smallest change to DL4S is an optional
// requirement on EngineType with a default implementation (in a protocol extension) that composes the existing
// primitives, so CPUEngine and GPUEngine stay untouched; CUDAEngine overrides it:
public extension CUDAEngine {
    /// ScaledDotProductAttention.swift:43-64 in one call. `keyLengths` / `causal` carry the masks of
    /// makeEncoderMasks / makeDecoderMasks (TransformerUtil.swift:29-50) without building them.
    static func scaledDotProductAttention(q: ShapedBuffer<Float, CUDA>, k: ShapedBuffer<Float, CUDA>, v: ShapedBuffer<Float, CUDA>,
                                          temperature: Float, keyLengths: Buffer<Int32, CUDA>?, causal: Bool,
                                          result: ShapedBuffer<Float, CUDA>) {
        let (B, H, Sq, dk) = (q.shape[0], q.shape[1], q.shape[2], q.shape[3]), Sk = k.shape[2], dv = v.shape[3]
        let lens = keyLengths?.memory.pointer?.assumingMemoryBound(to: Int32.self)
        if Sq == 1 && !causal {
            check(dl4s_cuda_sdpa_decode(q.values.memory.floats(), k.values.memory.floats(), v.values.memory.floats(), Int64(B), Int64(H),
                                        Int64(Sk), Int64(dk), Int64(dv), temperature, lens, result.values.memory.floats()))
        } else {
            check(dl4s_cuda_sdpa_forward(q.values.memory.floats(), k.values.memory.floats(), v.values.memory.floats(), Int64(B), Int64(H),
                                         Int64(Sq), Int64(Sk), Int64(dk), Int64(dv), temperature, lens, causal ? 1 : 0, nil, nil,
                                         result.values.memory.floats(), CUDA.precision))
        }
    }
    /// Gradients of the call above for the upstream gradient `dOut` (the backpropagate closures of the fused
    /// attention tensor): dq, dk, dv in one call, probabilities recomputed.
    static func scaledDotProductAttentionBackward(q: ShapedBuffer<Float, CUDA>, k: ShapedBuffer<Float, CUDA>, v: ShapedBuffer<Float, CUDA>,
                                                  dOut: ShapedBuffer<Float, CUDA>, temperature: Float,
                                                  keyLengths: Buffer<Int32, CUDA>?, causal: Bool,
                                                  dq: ShapedBuffer<Float, CUDA>, dk: ShapedBuffer<Float, CUDA>, dv: ShapedBuffer<Float, CUDA>) {
        let (B, H, Sq, dkk) = (q.shape[0], q.shape[1], q.shape[2], q.shape[3]), Sk = k.shape[2], dvv = v.shape[3]
        check(dl4s_cuda_sdpa_backward(q.values.memory.floats(), k.values.memory.floats(), v.values.memory.floats(),
                                      dOut.values.memory.floats(), Int64(B), Int64(H), Int64(Sq), Int64(Sk), Int64(dkk), Int64(dvv),
                                      temperature, keyLengths?.memory.pointer?.assumingMemoryBound(to: Int32.self), causal ? 1 : 0,
                                      nil, nil, dq.values.memory.floats(), dk.values.memory.floats(), dv.values.memory.floats(),
                                      CUDA.precision))
    }
    // multiHeadAttentionForward -> dl4s_cuda_mha_forward, layerNorm -> dl4s_cuda_layernorm (backward:
    // dl4s_cuda_layernorm_backward), feedForward -> dl4s_cuda_ffn_forward, encoderForward -> dl4s_cuda_encoder_forward
    // (or dl4s_cuda_encoder_prepare once + dl4s_cuda_encoder_forward_prepared per call for fixed weights),
    // decoderForward -> dl4s_cuda_decoder_forward, prepareInputs -> dl4s_cuda_embed_positional, the output head of
    // Transformer.callAsFunction -> dl4s_cuda_output_head, greedy decoding -> dl4s_cuda_transformer_greedy_decode,
    // Dropout -> dl4s_cuda_set_dropout(rate, seed) before the fused calls: same pattern.

    /// MultiHeadAttention whose heads are spread over the ranks of a communicator (one process per GPU). The library
    /// issues the all-gather itself; `CUDA.joinCommunicator(rank:world:id:)` wraps dl4s_cuda_comm_unique_id /
    /// dl4s_cuda_comm_init. `wq/wk/wv` are this rank's column slices, `result` the batch rows this rank owns
    /// (dl4s_cuda_mha_sharded_plan says which).
    static func multiHeadAttentionSharded(x: ShapedBuffer<Float, CUDA>, heads: Int, keyDim: Int, valueDim: Int,
                                          wq: ShapedBuffer<Float, CUDA>, wk: ShapedBuffer<Float, CUDA>, wv: ShapedBuffer<Float, CUDA>,
                                          wo: ShapedBuffer<Float, CUDA>, normScale: ShapedBuffer<Float, CUDA>, normShift: ShapedBuffer<Float, CUDA>,
                                          keyLengths: Buffer<Int32, CUDA>?, causal: Bool, chunks: Int, result: ShapedBuffer<Float, CUDA>) {
        let (B, S, D) = (x.shape[0], x.shape[1], x.shape[2])
        check(dl4s_cuda_mha_forward_sharded(x.values.memory.floats(), Int64(B), Int64(S), Int64(D), Int64(heads), Int64(keyDim),
                                            Int64(valueDim), wq.values.memory.floats(), wk.values.memory.floats(),
                                            wv.values.memory.floats(), wo.values.memory.floats(), normScale.values.memory.floats(),
                                            normShift.values.memory.floats(),
                                            keyLengths?.memory.pointer?.assumingMemoryBound(to: Int32.self), causal ? 1 : 0,
                                            result.values.memory.floats(), CUDA.precision, Int32(chunks)))
    }

    /// One step of incremental decoding. `kCache` / `vCache` are [B, H, maxLength, d]; `lengths` holds the tokens
    /// cached per sequence and is advanced by the caller after the call.
    static func decodeStep(x: ShapedBuffer<Float, CUDA>, heads: Int, keyDim: Int, valueDim: Int,
                           wq: ShapedBuffer<Float, CUDA>, wk: ShapedBuffer<Float, CUDA>, wv: ShapedBuffer<Float, CUDA>,
                           wo: ShapedBuffer<Float, CUDA>, normScale: ShapedBuffer<Float, CUDA>, normShift: ShapedBuffer<Float, CUDA>,
                           kCache: ShapedBuffer<Float, CUDA>, vCache: ShapedBuffer<Float, CUDA>,
                           lengths: ShapedBuffer<Int32, CUDA>, result: ShapedBuffer<Float, CUDA>) {
        let (B, D) = (x.shape[0], x.shape[1])
        check(dl4s_cuda_mha_decode_step(x.values.memory.floats(), Int64(B), Int64(D), Int64(heads), Int64(keyDim), Int64(valueDim),
                                        wq.values.memory.floats(), wk.values.memory.floats(), wv.values.memory.floats(),
                                        wo.values.memory.floats(), normScale.values.memory.floats(), normShift.values.memory.floats(),
                                        kCache.values.memory.floats(), vCache.values.memory.floats(), Int64(kCache.shape[2]),
                                        lengths.values.memory.pointer?.assumingMemoryBound(to: Int32.self),
                                        result.values.memory.floats()))
    }
}
#endif
