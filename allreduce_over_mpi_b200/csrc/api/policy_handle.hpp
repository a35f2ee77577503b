// The C handle of a selection policy (ft_policy in flextree.h), shared by the host API and the
// communicator runtime, which owns one per communicator.
#pragma once
#include "../planner/policy.hpp"
#include "flextree.h"

struct ft_policy {
  ft::Policy p;
  explicit ft_policy(int world) : p(world) {}
};

// C form of a policy answer.
void ft_policy_fill_choice(const ft::PolicyChoice& c, ft_choice* out);
