import CMfb200

/// Drop-in for the reference's `MoE` wrapper (Sources/Mference/Kernels/MoE/MoE.swift): same method names and argument
/// meaning; a Metal buffer + offset becomes a device pointer, the command buffer a CUDA stream.
public final class MoE {
    private var handle: OpaquePointer?
    public let d: Int, f: Int, numExperts: Int, topK: Int

    /// MoE.init(context:siluActivation:specializedD:F:NumExperts:TopK:) (MoE.swift:65-70).  `maxTokens` sizes the
    /// scratch arena (rows per call), `maxLayers` the per-layer tables of `encodeStack`.
    public init(siluActivation: Bool, specializedD d: Int, specializedF f: Int, specializedNumExperts e: Int,
                specializedTopK k: Int, bits: Int = 4, sharedBits: Int = 4, maxTokens: Int = 64, maxLayers: Int = 64,
                tensorCorePrefill: Bool = false) throws {
        self.d = d; self.f = f; self.numExperts = e; self.topK = k
        var cfg = mfb_moe_config()
        cfg.d = UInt32(d); cfg.f = UInt32(f); cfg.num_experts = UInt32(e); cfg.top_k = UInt32(k)
        cfg.bits = UInt32(bits); cfg.shared_bits = UInt32(sharedBits); cfg.group_size = 64
        cfg.scale_dtype = UInt32(MFB_DT_BF16)        // .gturbo files carry bf16 scales (Quantization.swift:32-45)
        cfg.x_dtype = UInt32(MFB_DT_F16)             // the reference's activations are half
        cfg.activation = UInt32(siluActivation ? MFB_ACT_SILU : MFB_ACT_GELU_TANH)
        cfg.router_mode = UInt32(MFB_ROUTER_SOFTMAX_TOPK); cfg.route_scale = 1; cfg.rms_eps = 1e-6
        cfg.max_tokens = UInt32(maxTokens); cfg.max_layers = UInt32(maxLayers)
        cfg.flags = tensorCorePrefill ? UInt32(MFB_FLAG_PREFILL_TENSOR_CORE) : 0
        try mfbCheck(mfb_moe_create(&cfg, &handle))
    }

    deinit { mfb_moe_destroy(handle) }

    /// encodeRouterGemma4 (MoE.swift:153-188): top-k expert indices and fp16 routing weights of `rows` token rows.  An
    /// INT8 gate is taken from `weights.router_scales` / `router_biases` when they are set.
    public func encodeRouterGemma4(stream: MfbStream, weights: inout LayerWeights, hidden: UnsafeRawPointer,
                                   hiddenStrideElements: Int? = nil, rows: Int = 1,
                                   outIndices: UnsafeMutablePointer<UInt32>, outWeights: UnsafeMutablePointer<UInt16>) throws {
        try mfbCheck(mfb_router_topk(handle, stream, hidden, UInt32(hiddenStrideElements ?? d), UInt32(rows), &weights,
                                     outIndices, outWeights))
    }

    /// encodeSlotLookup (MoE.swift:302-330).
    public func encodeSlotLookup(stream: MfbStream, indices: UnsafePointer<UInt32>, rows: Int, slotTable: UnsafePointer<Int16>,
                                 slotStride: UInt64, outOffsets: UnsafeMutablePointer<UInt64>,
                                 outAllHit: UnsafeMutablePointer<UInt32>) throws {
        try mfbCheck(mfb_slot_lookup(handle, stream, indices, UInt32(rows), slotTable, slotStride, outOffsets, outAllHit))
    }

    /// encodeRoutedPersistentPhase1(Subset)U16Load (MoE.swift:220-298) plus the down projections of the chosen rank
    /// slots; `activeSlots == nil` runs all of them.
    public func encodeRoutedExperts(stream: MfbStream, weights: inout LayerWeights, x: UnsafeRawPointer, rows: Int,
                                    indices: UnsafePointer<UInt32>, routingWeights: UnsafePointer<UInt16>,
                                    activeSlots: [UInt32]? = nil, withShared: Bool = true) throws {
        let rc: Int32
        if let slots = activeSlots {
            rc = slots.withUnsafeBufferPointer {
                mfb_moe_experts(handle, stream, &weights, x, UInt32(d), UInt32(rows), indices, routingWeights, $0.baseAddress,
                                UInt32(slots.count), withShared ? 1 : 0)
            }
        } else {
            rc = mfb_moe_experts(handle, stream, &weights, x, UInt32(d), UInt32(rows), indices, routingWeights, nil, 0, withShared ? 1 : 0)
        }
        try mfbCheck(rc)
    }

    /// encodeRoutedPersistentPhase2Reduce (MoE.swift:400-440): residual first, shared expert, ranks ascending.
    public func encodeRoutedPersistentPhase2Reduce(stream: MfbStream, rows: Int, routingWeights: UnsafePointer<UInt16>,
                                                   withShared: Bool, residual: UnsafeRawPointer?, y: UnsafeMutableRawPointer) throws {
        try mfbCheck(mfb_moe_combine(handle, stream, UInt32(rows), routingWeights, withShared ? 1 : 0, residual, y))
    }

    /// Phase 1, phase 2 and the reduce in one call (the all-hit path of RealForwardRunner.produceToken).
    public func encodeDecode(stream: MfbStream, weights: inout LayerWeights, x: UnsafeRawPointer, rows: Int,
                             indices: UnsafePointer<UInt32>, routingWeights: UnsafePointer<UInt16>, residual: UnsafeRawPointer?,
                             y: UnsafeMutableRawPointer) throws {
        try mfbCheck(mfb_moe_decode(handle, stream, &weights, x, UInt32(d), UInt32(rows), indices, routingWeights, residual, y))
    }

    /// One whole layer on the residual stream: hOut = hIn + MoE(RMSNorm(hIn)).
    public func encodeLayer(stream: MfbStream, weights: inout LayerWeights, hIn: UnsafeRawPointer, hOut: UnsafeMutableRawPointer,
                            rows: Int) throws {
        try mfbCheck(mfb_moe_layer(handle, stream, &weights, hIn, hOut, UInt32(rows)))
    }

    /// All layers of a decode step in one call (one cooperative kernel launch where the shape allows it).
    public func encodeStack(stream: MfbStream, layers: [LayerWeights], hidden: UnsafeMutableRawPointer, rows: Int) throws {
        try mfbCheck(layers.withUnsafeBufferPointer {
            mfb_moe_stack(handle, stream, $0.baseAddress, UInt32(layers.count), hidden, UInt32(rows))
        })
    }

    /// Reads and clears the device status word (a bounded wait that ran out is reported here, nothing hangs).
    public func deviceStatus(stream: MfbStream) throws -> UInt32 {
        var status: UInt32 = 0
        let rc = mfb_moe_device_status(handle, stream, &status)
        if rc != MFB_OK && rc != MFB_ERR_DEVICE_STATUS { try mfbCheck(rc) }
        return status
    }

    var raw: OpaquePointer? { handle }
}
