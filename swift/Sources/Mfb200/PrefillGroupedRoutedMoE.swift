import CMfb200

/// Drop-in for `PrefillMoEGrouping.groupTokenExpertPairs` on the device, `PrefillGroupedRoutedMoE.encodeStreamedBatched`
/// and `PrefillMoE.encodeReduceTokenMajor` (Sources/Mference/Kernels/Prefill/MoE/*.swift) over a `MoE` handle created
/// with `tensorCorePrefill: true`.
public final class PrefillGroupedRoutedMoE {
    private let moe: MoE

    public init(moe: MoE) { self.moe = moe }

    /// Sort of the routing table by (expert, token, rank): sorted pairs, per-expert offsets and counts, group list.
    public func encodeGroup(stream: MfbStream, indices: UnsafePointer<UInt32>, routingWeights: UnsafePointer<UInt16>, rows: Int,
                            sortedPairs: UnsafeMutablePointer<mfb_pair>, perExpertOffsets: UnsafeMutablePointer<UInt32>,
                            perExpertCounts: UnsafeMutablePointer<UInt32>, groups: UnsafeMutablePointer<mfb_group>,
                            groupCount: UnsafeMutablePointer<UInt32>) throws {
        try mfbCheck(mfb_moe_group(moe.raw, stream, indices, routingWeights, UInt32(rows), sortedPairs, perExpertOffsets,
                                   perExpertCounts, groups, groupCount))
    }

    /// encodeStreamedBatched (PrefillGroupedRoutedMoE.swift:391-466): partial[(token * topK + rank), :] for every pair.
    public func encodeStreamedBatched(stream: MfbStream, weights: inout LayerWeights, x: UnsafeRawPointer, rows: Int,
                                      sortedPairs: UnsafePointer<mfb_pair>, groups: UnsafePointer<mfb_group>,
                                      groupCount: UnsafePointer<UInt32>, partial: UnsafeMutablePointer<Float>) throws {
        try mfbCheck(mfb_moe_prefill_grouped(moe.raw, stream, &weights, x, UInt32(moe.d), UInt32(rows), sortedPairs, groups,
                                             groupCount, partial))
    }

    /// The Inkling batched expert application (inkling_prefill_expert_act + inkling_prefill_expert_down_accum,
    /// prefill.metal:654-746): acc (Float, rows x d, read and written) += the routed experts' rows, expert by expert in
    /// ascending expert order, with Float pair weights (rows x topK).
    public func encodeExpertAccumulateFloat32(stream: MfbStream, weights: inout LayerWeights, x: UnsafeRawPointer, rows: Int,
                                              sortedPairs: UnsafePointer<mfb_pair>, groups: UnsafePointer<mfb_group>,
                                              groupCount: UnsafePointer<UInt32>, pairWeights: UnsafePointer<Float>,
                                              acc: UnsafeMutablePointer<Float>) throws {
        try mfbCheck(mfb_moe_prefill_accumulate_f32(moe.raw, stream, &weights, x, UInt32(moe.d), UInt32(rows), sortedPairs, groups,
                                                    groupCount, pairWeights, acc))
    }

    /// encodeReduceTokenMajor (PrefillMoE.swift:11-38).
    public func encodeReduceTokenMajor(stream: MfbStream, partial: UnsafePointer<Float>, routingWeights: UnsafePointer<UInt16>,
                                       rows: Int, residual: UnsafeRawPointer?, y: UnsafeMutableRawPointer) throws {
        try mfbCheck(mfb_moe_reduce(moe.raw, stream, partial, routingWeights, UInt32(rows), residual, y))
    }

    /// The whole prefill layer of a chunk: norm, router, sort, grouped FFN with the shared expert, reduce.
    public func encodeLayer(stream: MfbStream, weights: inout LayerWeights, hIn: UnsafeRawPointer, hOut: UnsafeMutableRawPointer,
                            rows: Int) throws {
        try mfbCheck(mfb_moe_layer_prefill(moe.raw, stream, &weights, hIn, hOut, UInt32(rows)))
    }
}
