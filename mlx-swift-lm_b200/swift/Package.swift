// swift-tools-version: 5.9
// SwiftPM wiring for the B200 KV-cache library, laid out like the reference's
// MLXCXGrammar target (Package.swift:207-247 of mlx-swift-lm): a C target that
// only exposes the header + module map, and a Swift target on top of it.
// libkvcache_b200.so is built by mlx-swift-lm_b200/build.py (nvcc, sm_100a).
import PackageDescription

let package = Package(
    name: "KVCacheB200",
    products: [.library(name: "KVCacheB200", targets: ["KVCacheB200"])],
    targets: [
        .systemLibrary(name: "CKVCacheB200", path: "Sources/CKVCacheB200"),
        .target(
            name: "KVCacheB200",
            dependencies: ["CKVCacheB200"],
            path: "Sources/KVCacheB200",
            linkerSettings: [.linkedLibrary("kvcache_b200")]
        ),
    ]
)
