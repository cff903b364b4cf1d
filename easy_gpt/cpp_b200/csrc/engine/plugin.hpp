// What a plugin of the native engine includes.  A plugin is a shared library that adds parts (a mixer, a feed-forward,
// a norm, a position encoding, an embedding, a head) and architectures to the engine without a change to the engine's
// sources: it derives from the bases of parts_base.hpp, and exports
//
//     extern "C" void easygpt_register(easygpt::engine::PartRegistry* parts, easygpt::engine::ArchitectureRegistry* architectures);
//
// in which it puts factories into `parts` (parts->mixers["my_kind"] = ...) and builders into `architectures`
// (architectures->add("my_arch", builder), a function from the config.json object to a ModelSpec).  The engine loads it
// with ege_load_plugin (native.load_plugin in Python); from then on a model folder whose config.json names the
// architecture is built, loaded, cached, stepped, scheduled and replayed like any other.
//
// The interfaces, in short (parts_base.hpp has the details):
//   Part            tensor_requests() (names under its prefix, shapes), load(file, dtype), weight_bytes(), capturable()
//   Mixer           cache_need() -> paged keys/values (optionally a window), fixed-size state per request, or nothing;
//                   forward(ctx, input, cache view, follow) -> Delta [T, hidden] in ctx.dtype, taken from ctx.arena
//   FeedForward     forward(ctx, input, follow) -> Delta
//   Norm            forward(ctx, residual, delta, ..., out, ...): residual += delta, out = normalised rows
//   PositionEncoding  any of half_rotation(), apply_to_query_key(), add_to_embedding()
//   StepContext     the step's batch: token ids, positions, token -> entry map, entry starts / cached lengths / state slots
//                   (device arrays, and host twins outside captured steps), block tables and cache positions per group
#pragma once
#include "architectures.hpp"
#include "parts.hpp"
