// Stands in for the reference's src/ops.h where only its attention operators are used (namespace q27,
// src/ops.h:50-77): a translation unit that includes "ops.h" and calls kv_cache_bytes, attn_prep,
// attn_decode, attn_prefill, attn_decode_ref or attn_chunks compiles against this directory unchanged.
#pragma once
#include "ops_attn.h"
