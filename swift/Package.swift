// swift-tools-version: 5.9
// Linux host package: the reference's `TritonMetalCore` surface over libtmcuda.
//
// Mirrors the product shape of the reference's Package.swift (a library the Python shim
// and tmbench link against) with the Metal runtime replaced by the C-ABI CUDA library.
// Not compiled in this repository's CI: the build image has no Swift toolchain.
import PackageDescription

let package = Package(
    name: "TritonMetalCuda",
    products: [
        .library(name: "TritonMetalCore", targets: ["TritonMetalCore"]),
    ],
    targets: [
        // System-library target: module map + include/tm.h; links libtmcuda.so.
        .systemLibrary(name: "CTMCuda", path: "Sources/CTMCuda"),
        .target(name: "TritonMetalCore", dependencies: ["CTMCuda"]),
    ]
)
