// swift-tools-version: 6.1
// Drop-in layer for the reference engine: the same wrapper classes (MoE, PrefillGroupedRoutedMoE, ExpertSlotCache)
// over the C ABI of libmfb200.so.  The image this repository is built and tested in has no Swift toolchain, so these
// sources are NOT compiled or tested here; the C ABI they call is exercised through the same entry points by the
// Python host layer and its tests.
import PackageDescription

let package = Package(
    name: "Mfb200",
    products: [.library(name: "Mfb200", targets: ["Mfb200"])],
    targets: [
        .systemLibrary(name: "CMfb200", path: "Sources/CMfb200"),
        .target(name: "Mfb200", dependencies: ["CMfb200"], path: "Sources/Mfb200"),
    ]
)
