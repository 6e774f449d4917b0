import CMfb200

/// Drop-in for the expert-slot cache side of `PreadExpertStreamer`
/// (Sources/Mference/Infrastructure/Streaming/PreadExpertStreamer.swift): the same plan / execute / publish protocol over
/// a slab in HBM that is filled from pinned host memory instead of from SSD.
public final class ExpertSlotCache {
    public struct Plan {
        public let experts: [Int32]
        public var assignedSlots: [Int32]
        public var miss: [UInt8]
        public var hits: Int
    }

    private var pool: OpaquePointer?
    public let numExperts: Int, slotCount: Int

    public init(numExperts: Int, slotBytes: UInt64, slotCount: Int, lru: Bool = false) throws {
        self.numExperts = numExperts; self.slotCount = slotCount
        try mfbCheck(mfb_pool_create(UInt32(numExperts), slotBytes, UInt32(slotCount), lru ? UInt32(MFB_POOL_LRU) : UInt32(MFB_POOL_LFU),
                                     0, &pool))
    }

    deinit { mfb_pool_destroy(pool) }

    /// routedSlotMapBinding: slab, slot stride and the device-resident expert -> slot table, for `LayerWeights`.
    public func bind(into weights: inout LayerWeights) throws {
        var slab: UnsafeMutableRawPointer?
        var stride: UInt64 = 0
        var table: UnsafePointer<Int16>?
        try mfbCheck(mfb_pool_info(pool, &slab, &stride, &table))
        weights.pool = UnsafePointer(slab?.assumingMemoryBound(to: UInt8.self))
        weights.slot_stride = stride
        weights.slot_of = table
    }

    /// planExpertsCachedIfPossible (PreadExpertStreamer.swift:197-269): nil when the misses cannot be placed.
    public func planExpertsCachedIfPossible(_ experts: [Int32], avoidingSlots: [Int32] = []) throws -> Plan? {
        var slots = [Int32](repeating: -1, count: experts.count)
        var miss = [UInt8](repeating: 0, count: experts.count)
        var hits: UInt32 = 0
        let rc = mfb_pool_plan(pool, experts, UInt32(experts.count), avoidingSlots, UInt32(avoidingSlots.count), &slots, &miss, &hits)
        if rc == MFB_ERR_NO_SLOT { return nil }
        try mfbCheck(rc)
        return Plan(experts: experts, assignedSlots: slots, miss: miss, hits: Int(hits))
    }

    /// executeExpertCachePlan (PreadExpertStreamer.swift:271-302): one copy per miss from pinned host memory, then publish.
    public func executeExpertCachePlan(_ plan: Plan, stream: MfbStream, hostBlobs: [UnsafeRawPointer?], blobBytes: UInt64) throws {
        try mfbCheck(mfb_pool_fill_async(pool, stream, plan.experts, plan.assignedSlots, plan.miss, UInt32(plan.experts.count),
                                         hostBlobs, blobBytes))
        try mfbCheck(mfb_pool_publish(pool, stream, plan.experts, plan.assignedSlots, plan.miss, UInt32(plan.experts.count)))
    }

    /// reserveSpeculativeSlots (PreadExpertStreamer.swift:344-372).
    public func reserveSpeculativeSlots(experts: [Int32], keepEvictable: Int) throws -> [(expert: Int32, slot: Int32)] {
        var outE = [Int32](repeating: 0, count: experts.count), outS = [Int32](repeating: 0, count: experts.count)
        var n: UInt32 = 0
        try mfbCheck(mfb_pool_reserve_speculative(pool, experts, UInt32(experts.count), UInt32(max(0, keepEvictable)), &outE, &outS, &n))
        return (0..<Int(n)).map { (outE[$0], outS[$0]) }
    }

    /// noteAllHitUse (PreadExpertStreamer.swift:427-440).
    public func noteAllHitUse(experts: [Int32]) throws {
        try mfbCheck(mfb_pool_note_all_hit(pool, experts, UInt32(experts.count)))
    }
}
