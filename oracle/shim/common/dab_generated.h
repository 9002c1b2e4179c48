// TEST INFRASTRUCTURE ONLY (part of the parity oracle; never used by the product path).
// Shadows the reference's flatc-generated common/dab_generated.h so that dabnn/net.h
// (which only needs the name flatbnn::Model, net.h:10,56) compiles without the FlatBuffers
// C++ runtime, an empty un-vendored submodule in the reference checkout.
#pragma once
namespace flatbnn { struct Model; }
