// type_list::list<Ts...> and type_list::get_type<I, list>::type, the indexable list of weight
// formats the reference's sweep drivers iterate over (lib/type_list.hpp,
// Linear/test/benchmark.cu:35-41).
#pragma once
#include <cstddef>
#include <tuple>

namespace type_list {
template <typename... Ts> struct list {
    static_assert(sizeof...(Ts) > 0, "a type list holds at least one type");
    using as_tuple = std::tuple<Ts...>;
    static const auto size = sizeof...(Ts);
};
template <int Index, typename Container> struct get_type {
    static_assert(Index >= 0 && static_cast<std::size_t>(Index) < Container::size,
                  "type_list index out of range");
    using type = std::tuple_element_t<static_cast<std::size_t>(Index), typename Container::as_tuple>;
};
}  // namespace type_list
