import CMfb200

/// Status of a failed call with the library's text for the calling thread.
public enum Mfb200Error: Error {
    case status(code: Int32, text: String)
}

@inline(__always)
func mfbCheck(_ rc: Int32) throws {
    if rc != MFB_OK { throw Mfb200Error.status(code: rc, text: String(cString: mfb_last_error())) }
}

/// A CUDA stream handle as the C ABI takes it (the reference's MTLCommandBuffer).
public typealias MfbStream = UnsafeMutableRawPointer?

/// Device-resident weights of one layer: the fields of `mfb_layer_weights`, filled by whoever owns the expert pool
/// (ExpertSlotCache) and the resident tensors.
public typealias LayerWeights = mfb_layer_weights
